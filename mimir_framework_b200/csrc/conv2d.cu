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
    // (ci, ky, kx) of the chunk's first entry by division, of the other seven by stepping
    int ci = (c * 8) / kk, t = c * 8 - ci * kk;
    int ky = t / ks, kx = t - ky * ks;
    const int iy0 = oy * stride - pad, ix0 = ox * stride - pad;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v = 0.0f;
      if (c * 8 + j < k) {
        const int iy = iy0 + ky, ix = ix0 + kx;
        if (iy >= 0 && iy < h && ix >= 0 && ix < w) v = __ldg(xs + (static_cast<long long>(ci) * h + iy) * w + ix);
      }
      split_one(v, f16, hi[j], lo[j]);
      if (++kx == ks) {
        kx = 0;
        if (++ky == ks) { ky = 0; ++ci; }
      }
    }
    __nv_bfloat16* d = dst + r * kp + c * 8;
    *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(hi);
    if (planes == 2) *reinterpret_cast<uint4*>(d + plane_stride) = *reinterpret_cast<const uint4*>(lo);
  }
}

// The same rows from a staged input patch: a CTA owns I2C_TPX consecutive output pixels of one output row and a block of
// `cb` input channels (a multiple of 8, or all of them), loads the patch those pixels read - cb x ks rows of
// (I2C_TPX - 1) * stride + ks input pixels, coalesced - into shared memory once, and assembles the 16-byte chunks of its K
// range from there (consecutive threads: consecutive chunks of one pixel, i.e. contiguous stores).  The input is read
// once per channel block instead of once per K entry through the caches, and the index arithmetic is per chunk.
constexpr int I2C_TPX = 32;

__global__ void __launch_bounds__(256) im2col_tile_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ dst, long long rows,
                                                          int ic, int h, int w, int ks, int stride, int pad, int oh, int ow, int k,
                                                          int kp, int planes, int f16, int cb, int nblocks) {
  extern __shared__ float patch[];  // [cbn][ks][pw]
  const int ox0 = blockIdx.x * I2C_TPX, oy = blockIdx.y;
  const int smp = blockIdx.z / nblocks, blk = blockIdx.z - smp * nblocks;
  const int c0 = blk * cb, cbn = min(cb, ic - c0);
  const int kk = ks * ks, pw = (I2C_TPX - 1) * stride + ks;
  const int iy0 = oy * stride - pad, ix0 = ox0 * stride - pad;
  const float* xs = x + (static_cast<long long>(smp) * ic + c0) * h * w;
  for (int i = threadIdx.x; i < cbn * ks * pw; i += 256) {
    const int c = i / (ks * pw), r = i - c * (ks * pw);
    const int ky = r / pw, px = r - ky * pw;
    const int iy = iy0 + ky, ix = ix0 + px;
    patch[i] = (iy >= 0 && iy < h && ix >= 0 && ix < w) ? __ldg(xs + (static_cast<long long>(c) * h + iy) * w + ix) : 0.0f;
  }
  __syncthreads();
  // this block's chunks of a row: its channels' K range; the last block also writes the zero padding up to kp
  const int ch_lo = (c0 * kk) >> 3, ch_hi = (blk == nblocks - 1) ? (kp >> 3) : (((c0 + cbn) * kk) >> 3);
  const int nch = ch_hi - ch_lo, npx = min(I2C_TPX, ow - ox0);
  const long long plane_stride = rows * static_cast<long long>(kp);
  const long long row0 = (static_cast<long long>(smp) * oh + oy) * ow + ox0;
  for (int item = threadIdx.x; item < npx * nch; item += 256) {
    const int p = item / nch, chunk = ch_lo + (item - p * nch);
    const int kidx0 = chunk * 8 - c0 * kk;  // relative to this block's first channel
    int ci = kidx0 / kk, t = kidx0 - ci * kk;
    int ky = t / ks, kx = t - ky * ks;
    __align__(16) uint16_t hi[8];
    __align__(16) uint16_t lo[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float v = (ci < cbn) ? patch[(ci * ks + ky) * pw + p * stride + kx] : 0.0f;  // past the last channel: K padding
      split_one(v, f16, hi[j], lo[j]);
      if (++kx == ks) {
        kx = 0;
        if (++ky == ks) { ky = 0; ++ci; }
      }
    }
    __nv_bfloat16* d = dst + (row0 + p) * kp + chunk * 8;
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
  {
    // the staged form: channel blocks of a multiple of 8 (so that every block starts on a chunk boundary) within 48 KB
    static const bool off = [] { const char* e = getenv("MIMIR_B200_IM2COL_TILED"); return e && e[0] == '0'; }();
    const int pw = (I2C_TPX - 1) * stride + ks;
    const long long per_ch = static_cast<long long>(ks) * pw * 4;
    int cb = static_cast<int>(std::min<long long>(ic, (48 * 1024) / per_ch));
    if (cb < ic) cb &= ~7;
    const int nblocks = cb > 0 ? (ic + cb - 1) / cb : 0;
    if (!off && cb > 0 && static_cast<long long>(batch) * nblocks <= 65535 && oh <= 65535) {
      dim3 grid((ow + I2C_TPX - 1) / I2C_TPX, oh, batch * nblocks);
      im2col_tile_kernel<<<grid, 256, static_cast<size_t>(cb) * per_ch, st>>>(x, dst, rows, ic, h, w, ks, stride, pad, oh, ow, k, kp, planes,
                                                                              plane_format() == PLANES_F16, cb, nblocks);
      MB_CUDA(cudaGetLastError());
      count_launch();
      return MIMIR_B200_OK;
    }
  }
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

__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gmem_src, bool valid) {
  // 16 bytes, or 16 zero bytes when !valid (source size 0: nothing is read)
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(gmem_src), "r"(valid ? 16 : 0)
               : "memory");
}

__global__ void __launch_bounds__(256, 3) nchw_to_padded_nhwc_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ dst,
                                                                  int c, int h, int w, int pad, int planes, long long plane_stride,
                                                                  const PreNorm pre, int f16, int up) {
  __shared__ float tile[TP_C][TP_X + 1];
  const int hp = h + 2 * pad, wp = w + 2 * pad;
  const int cb = blockIdx.x * TP_C;
  const int yp = blockIdx.y;
  const int n = blockIdx.z;
  const int y = yp - pad;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool row_in = y >= 0 && y < h;
  // up: the source is the half-size image, a source pixel feeds a 2 x 2 block
  const int sh_ = up ? h >> 1 : h, sw_ = up ? w >> 1 : w;
  const float* src = x + ((static_cast<long long>(n) * c + cb) * sh_ + (row_in ? (up ? y >> 1 : y) : 0)) * sw_;
  const long long ch_stride = static_cast<long long>(sh_) * sw_;
  // scale / shift of the CTA's 64 channels once, in shared memory; a thread's 16 elements of a tile belong to 16 fixed
  // channels ((tid >> 6) + 4 i), so it keeps those 16 pairs in registers for every tile of the row
  __shared__ float2 s_aff[TP_C];
  float sc[16], sh[16];
  if (pre.stats != nullptr) {
    if (threadIdx.x < TP_C) {
      const int ch = cb + threadIdx.x;
      float2 a = make_float2(0.0f, 0.0f);
      if (ch < c) {
        const float* st = pre.stats + (static_cast<long long>(n) * pre.groups + ch / (c / pre.groups)) * 2;
        const float mean = __ldg(st), inv = __ldg(st + 1);
        const float g = pre.gamma != nullptr ? __ldg(pre.gamma + ch) : 1.0f;
        const float b = (pre.gamma != nullptr && pre.beta != nullptr) ? __ldg(pre.beta + ch) : 0.0f;
        a = make_float2(inv * g, b - mean * inv * g);
      }
      s_aff[threadIdx.x] = a;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 a = s_aff[(threadIdx.x >> 6) + 4 * i];
      sc[i] = a.x; sh[i] = a.y;
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
      v[i] = (row_in && xs >= 0 && xs < w && cb + cc < c) ? __ldg(src + cc * ch_stride + (up ? xs >> 1 : xs)) : 0.0f;
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

// The same layout pass with 16-byte accesses on both sides, for widths that are a multiple of 4 and channel counts that
// are a multiple of 8: tiles are aligned to the INPUT pixels (so a thread's float4 is four consecutive pixels of one
// channel), the shift by the padding happens on the way out, where a thread owns eight consecutive channels of one pixel
// (one 16-byte store per plane).  The padding ring is written as zeros by the CTAs of the border rows and by the first
// and last tile of every interior row.
__global__ void __launch_bounds__(256) nchw_to_padded_nhwc_vec_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ dst,
                                                                      int c, int h, int w, int pad, int planes, long long plane_stride,
                                                                      const PreNorm pre, int f16, int up) {
  __shared__ float tile[TP_C][TP_X + 1];
  __shared__ float2 s_aff[TP_C];
  const int hp = h + 2 * pad, wp = w + 2 * pad;
  const int cb = blockIdx.x * TP_C;
  const int yp = blockIdx.y;
  const int n = blockIdx.z;
  const int y = yp - pad;
  const long long row_o = (static_cast<long long>(n) * hp + yp) * wp;  // first padded pixel of this output row
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  auto store8 = [&](long long pixel, int ch, const uint4& hi, const uint4& lo) {
    __nv_bfloat16* o = dst + pixel * c + ch;
    *reinterpret_cast<uint4*>(o) = hi;
    if (planes == 2) *reinterpret_cast<uint4*>(o + plane_stride) = lo;
  };
  if (y < 0 || y >= h) {  // a border row: zeros
    for (int r = threadIdx.x; r < wp * (TP_C / 8); r += 256) {
      const int xp = r >> 3, ch = cb + 8 * (r & 7);
      if (ch < c) store8(row_o + xp, ch, zero4, zero4);
    }
    return;
  }
  for (int r = threadIdx.x; r < 2 * pad * (TP_C / 8); r += 256) {  // the row's left and right padding pixels
    const int q = r >> 3, ch = cb + 8 * (r & 7);
    const int xp = q < pad ? q : w + q;  // q - pad + (w + pad)
    if (ch < c) store8(row_o + xp, ch, zero4, zero4);
  }
  // up: the source is the half-size image; four consecutive output pixels are two source pixels, each used twice
  const int sh_ = up ? h >> 1 : h, sw_ = up ? w >> 1 : w;
  const float* src = x + ((static_cast<long long>(n) * c + cb) * sh_ + (up ? y >> 1 : y)) * sw_;
  const long long ch_stride = static_cast<long long>(sh_) * sw_;
  // a thread's four float4 of a tile belong to the channels (tid >> 4) + 16 i
  float sc[4], sh[4];
  if (pre.stats != nullptr) {
    if (threadIdx.x < TP_C) {
      const int ch = cb + threadIdx.x;
      float2 a = make_float2(0.0f, 0.0f);
      if (ch < c) {
        const float* st = pre.stats + (static_cast<long long>(n) * pre.groups + ch / (c / pre.groups)) * 2;
        const float mean = __ldg(st), inv = __ldg(st + 1);
        const float g = pre.gamma != nullptr ? __ldg(pre.gamma + ch) : 1.0f;
        const float b = (pre.gamma != nullptr && pre.beta != nullptr) ? __ldg(pre.beta + ch) : 0.0f;
        a = make_float2(inv * g, b - mean * inv * g);
      }
      s_aff[threadIdx.x] = a;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = s_aff[(threadIdx.x >> 4) + 16 * i];
      sc[i] = a.x; sh[i] = a.y;
    }
  }
  for (int x0 = 0; x0 < w; x0 += TP_X) {
    float4 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int cc = (threadIdx.x >> 4) + 16 * i, xs = x0 + 4 * (threadIdx.x & 15);
      if (xs < w && cb + cc < c) {
        if (up) {
          const float2 t = __ldg(reinterpret_cast<const float2*>(src + cc * ch_stride + (xs >> 1)));
          v[i] = make_float4(t.x, t.x, t.y, t.y);
        } else {
          v[i] = __ldg(reinterpret_cast<const float4*>(src + cc * ch_stride + xs));
        }
      } else {
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    if (pre.stats != nullptr) {  // GroupNorm (+ SiLU) of the producer applied here
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float* e = reinterpret_cast<float*>(&v[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float r = fmaf(e[j], sc[i], sh[i]);
          if (pre.act == MIMIR_B200_ELT_SILU) r = r * __fdividef(1.0f, 1.0f + __expf(-r));
          e[j] = r;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float* t = &tile[(threadIdx.x >> 4) + 16 * i][4 * (threadIdx.x & 15)];
      t[0] = v[i].x; t[1] = v[i].y; t[2] = v[i].z; t[3] = v[i].w;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = threadIdx.x + 256 * i;
      const int xx = r >> 3, ch8 = 8 * (r & 7);
      if (x0 + xx < w && cb + ch8 < c) {
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) split_pair(tile[ch8 + 2 * j][xx], tile[ch8 + 2 * j + 1][xx], f16, hi[j], lo[j]);
        store8(row_o + pad + x0 + xx, cb + ch8, make_uint4(hi[0], hi[1], hi[2], hi[3]), make_uint4(lo[0], lo[1], lo[2], lo[3]));
      }
    }
    __syncthreads();
  }
}

// The streaming form of the same pass: a CTA owns LR_ROWS output rows of one sample and 64 channels and walks their tiles
// (64 channels x 64 pixels) as one sequence; the source of tile t + 1 is on its way into the second shared-memory buffer
// (16-byte cp.async, zero-filled past the image or the channel count) while tile t is normalised, split and stored, so the
// loads of a CTA never stop for its stores (the kernel above alternates the two and sat at 30 % issue utilisation with
// 15 stall cycles per issue on memory).  The tile is stored with its 16-byte column groups XOR-ed with the channel's octet:
// the eight lanes that write one pixel's 64 channels then read eight different bank groups.  UP = 1 gathers the 2 x 2 nearest
// upsample: a tile's source is 32 pixels of the half-size row, each read twice.
constexpr int LR_ROWS = 4, LR_TS = TP_X + 4;
template <int UP>
__global__ void __launch_bounds__(256, 5) nchw_to_padded_nhwc_stream_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ dst,
                                                                           int c, int h, int w, int pad, int planes,
                                                                           long long plane_stride, const PreNorm pre, int f16) {
  __shared__ __align__(16) float tile[2][TP_C][LR_TS];
  const int hp = h + 2 * pad, wp = w + 2 * pad;
  const int cb = blockIdx.x * TP_C, n = blockIdx.z;
  const int yp0 = blockIdx.y * LR_ROWS, yp1 = min(hp, yp0 + LR_ROWS);
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  auto store8 = [&](long long pixel, int ch, const uint4& hi, const uint4& lo) {
    __nv_bfloat16* o = dst + pixel * c + ch;
    *reinterpret_cast<uint4*>(o) = hi;
    if (planes == 2) *reinterpret_cast<uint4*>(o + plane_stride) = lo;
  };
  // the padding ring of these rows: whole border rows, and the left and right padding pixels of the interior ones
  for (int yp = yp0; yp < yp1; ++yp) {
    const long long row_o = (static_cast<long long>(n) * hp + yp) * wp;
    const bool border = yp < pad || yp >= h + pad;
    const int npix = border ? wp : 2 * pad;
    for (int r = threadIdx.x; r < npix * (TP_C / 8); r += 256) {
      const int q = r >> 3, ch = cb + 8 * (r & 7);
      const int xp = border ? q : (q < pad ? q : w + q);
      if (ch < c) store8(row_o + xp, ch, zero4, zero4);
    }
  }
  const int y_lo = max(yp0, pad), y_hi = min(yp1, h + pad);  // interior rows (padded numbering)
  if (y_lo >= y_hi) return;
  const int tiles_x = (w + TP_X - 1) / TP_X, ntiles = (y_hi - y_lo) * tiles_x;
  const int sh_ = UP ? h >> 1 : h, sw_ = UP ? w >> 1 : w;
  const float* src_n = x + (static_cast<long long>(n) * c + cb) * sh_ * sw_;
  const long long ch_stride = static_cast<long long>(sh_) * sw_;
  // this thread's eight channels on the way out, and their GroupNorm scale / shift
  const int ch8 = 8 * (threadIdx.x & 7), oct = threadIdx.x & 7;
  float sc[8], sf[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) { sc[k] = 1.0f; sf[k] = 0.0f; }
  if (pre.stats != nullptr) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int ch = cb + ch8 + k;
      if (ch < c) {
        const float* st = pre.stats + (static_cast<long long>(n) * pre.groups + ch / (c / pre.groups)) * 2;
        const float mean = __ldg(st), inv = __ldg(st + 1);
        const float g = pre.gamma != nullptr ? __ldg(pre.gamma + ch) : 1.0f;
        const float b = (pre.gamma != nullptr && pre.beta != nullptr) ? __ldg(pre.beta + ch) : 0.0f;
        sc[k] = inv * g;
        sf[k] = b - mean * inv * g;
      }
    }
  }
  constexpr int SRC_CHUNKS = UP ? TP_X / 8 : TP_X / 4;  // 16-byte chunks of one channel's tile source
  auto issue = [&](int t) {
    const int ty = t / tiles_x, x0 = (t - ty * tiles_x) * TP_X;
    const int y = y_lo + ty - pad;
    const float* srow = src_n + static_cast<long long>(UP ? y >> 1 : y) * sw_ + (UP ? x0 >> 1 : x0);
    float(*buf)[LR_TS] = tile[t & 1];
#pragma unroll
    for (int i = 0; i < TP_C * SRC_CHUNKS / 256; ++i) {
      const int idx = threadIdx.x + 256 * i;
      const int cc = idx / SRC_CHUNKS, q = idx - cc * SRC_CHUNKS;
      const int xs = (UP ? x0 >> 1 : x0) + 4 * q;
      const bool ok = xs < sw_ && cb + cc < c;
      cp_async16_zfill(&buf[cc][4 * (q ^ ((cc >> 3) & 7))], ok ? srow + cc * ch_stride + 4 * q : x, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  issue(0);
  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) issue(t + 1);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    const int ty = t / tiles_x, x0 = (t - ty * tiles_x) * TP_X;
    const long long row_o = (static_cast<long long>(n) * hp + y_lo + ty) * wp + pad + x0;
    const float(*buf)[LR_TS] = tile[t & 1];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int xx = (threadIdx.x + 256 * i) >> 3;
      if (x0 + xx < w && cb + ch8 < c) {
        const int sx = UP ? xx >> 1 : xx;
        const int col = 4 * ((sx >> 2) ^ oct) + (sx & 3);  // (ch8 + k) >> 3 = oct for every k
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = buf[ch8 + k][col];
        if (pre.stats != nullptr) {  // GroupNorm (+ SiLU) of the producer applied here
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            float r = fmaf(v[k], sc[k], sf[k]);
            if (pre.act == MIMIR_B200_ELT_SILU) r = r * __fdividef(1.0f, 1.0f + __expf(-r));
            v[k] = r;
          }
        }
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) split_pair(v[2 * j], v[2 * j + 1], f16, hi[j], lo[j]);
        store8(row_o + xx, cb + ch8, make_uint4(hi[0], hi[1], hi[2], hi[3]), make_uint4(lo[0], lo[1], lo[2], lo[3]));
      }
    }
    __syncthreads();  // the buffer is refilled by the copy issued at the top of the next iteration
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
                                     cudaStream_t st, const PreNorm& pre, int up) {
  if (batch <= 0 || c <= 0 || h <= 0 || w <= 0 || pad < 0) return fail(MIMIR_B200_E_INVALID, "Conv2d: bad activation shape");
  if (up && ((h | w) & 1)) return fail(MIMIR_B200_E_INVALID, "Conv2d: an upsampled input needs even dimensions");
  const int hp = h + 2 * pad, wp = w + 2 * pad;
  if (hp > 65535 || batch > 65535) return fail(MIMIR_B200_E_UNSUPPORTED, "Conv2d: image too tall for the layout kernel");
  dim3 grid((c + TP_C - 1) / TP_C, hp, batch);
  if (pre.stats != nullptr && (pre.groups <= 0 || c % pre.groups != 0)) return fail(MIMIR_B200_E_INVALID, "Conv2d: bad fused GroupNorm");
  static const bool no_vec = [] { const char* e = getenv("MIMIR_B200_LAYOUT_VEC"); return e && e[0] == '0'; }();
  const long long plane_stride = static_cast<long long>(batch) * hp * wp * c;
  const bool vec = !no_vec && (w & 3) == 0 && (c & 7) == 0 && (plane_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
  // rows streamed through a double buffer (MIMIR_B200_LAYOUT_STREAM=0 turns it off); the upsampling form needs the half-size
  // rows to be whole 16-byte chunks too
  static const bool no_stream = [] { const char* e = getenv("MIMIR_B200_LAYOUT_STREAM"); return e && e[0] == '0'; }();
  if (vec && !no_stream && (!up || ((w >> 1) & 3) == 0) && (hp + LR_ROWS - 1) / LR_ROWS <= 65535) {
    dim3 sgrid((c + TP_C - 1) / TP_C, (hp + LR_ROWS - 1) / LR_ROWS, batch);
    const int f16 = plane_format() == PLANES_F16;
    if (up) nchw_to_padded_nhwc_stream_kernel<1><<<sgrid, 256, 0, st>>>(x, dst, c, h, w, pad, planes, plane_stride, pre, f16);
    else nchw_to_padded_nhwc_stream_kernel<0><<<sgrid, 256, 0, st>>>(x, dst, c, h, w, pad, planes, plane_stride, pre, f16);
  } else if (vec)
    nchw_to_padded_nhwc_vec_kernel<<<grid, 256, 0, st>>>(x, dst, c, h, w, pad, planes, plane_stride, pre, plane_format() == PLANES_F16, up);
  else
    nchw_to_padded_nhwc_kernel<<<grid, 256, 0, st>>>(x, dst, c, h, w, pad, planes, plane_stride, pre, plane_format() == PLANES_F16, up);
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

// ---------------------------------------------------------------------------------------------
// Convolutions with very few output channels (an RGB head: 128 -> 3): on the tensor core a 128-row weight tile would be
// all padding, and the layer is bound by reading its input once.  Direct fp32 convolution instead: a CTA owns a
// 128 x 8 pixel tile of one sample, stages the input tile (with its halo) for four channels at a time in shared memory,
// and every thread accumulates all output channels of its four pixels in the reference's order (ic, kh, kw ascending,
// Model.cpp:5005-5032) with FMAs.  No operand planes, no layout pass.
// ---------------------------------------------------------------------------------------------
namespace mb {
namespace {

constexpr int SO_TX = 32, SO_TY = 8, SO_PX = 4, SO_CC = 2, SO_NBUF = 2, SO_MAX_OC = 8, SO_MAX_KS = 7;
constexpr int so_rows(int oc) { return oc <= 4 ? 2 : 1; }  // output rows per thread: as many as the accumulators leave registers for

// A thread owns SO_PX consecutive pixels of R consecutive rows.  Every input row segment it reads from shared memory
// feeds all taps of up to R output rows, and the weights of one (channel, kernel row) come as broadcast 16-byte loads,
// so the FMA pipe and not the shared-memory pipe sets the pace.  The input tile and the weights of the next SO_CC
// channels arrive through cp.async (4-byte copies, plain zero stores for the padding ring) into the next slot of a
// ring of SO_NBUF buffers while the current channels are being consumed: one barrier per chunk, no registers spent on staging.
// Each output element accumulates over (ic, kh, kw) ascending: the reference's order (Model.cpp:5005-5032).
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gmem_src)
               : "memory");
}


// VEC = 0: tile rows of TW = 128 + KS - 1 pixels copied element by element, a pad word after every SO_PX pixels (the lanes of a
//          warp then read their segments SO_PX + 1 words apart: no bank conflicts).  Any image width and alignment.
// VEC = 1: image rows that are whole 16-byte chunks (width a multiple of 4, aligned base): a tile row is the 136 pixels from
//          x0 - 4, copied as 34 aligned 16-byte chunks (zero-filled outside the image); a lane reads its four pixels with one
//          128-bit load and takes the halo from its neighbours' registers.
template <int KS, int R, int VEC>
struct SmallOcGeom {
  static constexpr int PAD = KS / 2, TW = SO_TX * SO_PX + KS - 1, TH = SO_TY * R + KS - 1, SEG = SO_PX + KS - 1;
  static constexpr int TWV = SO_TX * SO_PX + 8, CHUNKS = TWV / 4;
  static constexpr int TWP = VEC ? TWV : TW + TW / SO_PX + 1;  // row stride in shared memory
  static constexpr int TILE = SO_CC * TH * TWP, WOFF = (SO_NBUF * TILE + 3) & ~3;
};

template <int OC, int KS, int R, int VEC>
__global__ void __launch_bounds__(SO_TX * SO_TY) conv_small_oc_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                       float* __restrict__ y, const float* __restrict__ residual, int ic,
                                                                       int h, int wd, int act) {
  using G = SmallOcGeom<KS, R, VEC>;
  constexpr int PAD = G::PAD, TW = G::TW, TH = G::TH, TWP = G::TWP, TILE = G::TILE, SEG = G::SEG, KK = KS * KS;
  constexpr int WROW = (KS * OC + 3) & ~3;  // the weights of one (channel, kernel row) as [kw][o], padded to whole float4s
  constexpr int WCH = SO_CC * KS * WROW;
  extern __shared__ __align__(16) float so_smem[];  // [SO_NBUF][TILE] input tiles, then (16-byte aligned) [SO_NBUF][WCH] weights
  const int n = blockIdx.z;
  const int x0 = blockIdx.x * (SO_TX * SO_PX), y0 = blockIdx.y * (SO_TY * R);
  const int tx = threadIdx.x & (SO_TX - 1), ty = threadIdx.x / SO_TX;
  const float* xs = x + static_cast<long long>(n) * ic * h * wd;
  float acc[OC][R][SO_PX];
#pragma unroll
  for (int o = 0; o < OC; ++o)
#pragma unroll
    for (int j = 0; j < R; ++j)
#pragma unroll
      for (int q = 0; q < SO_PX; ++q) acc[o][j][q] = 0.0f;
  for (int i = threadIdx.x; i < SO_NBUF * WCH; i += SO_TX * SO_TY) so_smem[G::WOFF + i] = 0.0f;  // the float4 padding is read, never used
  __syncthreads();
  // a lane copies the same columns of every tile row: their offsets and bounds once per thread
  constexpr int NX = (TW + SO_TX - 1) / SO_TX;
  int xsrc[NX], xdst[NX];  // xsrc < 0: outside the image (or past the tile): a zero is stored, or nothing
#pragma unroll
  for (int k = 0; k < NX; ++k) {
    const int xx = tx + k * SO_TX, gx = x0 - PAD + xx;
    xdst[k] = xx < TW ? xx + xx / SO_PX : -1;
    xsrc[k] = (xx < TW && gx >= 0 && gx < wd) ? gx : -1;
  }
  auto fetch = [&](int c0, int buf) {
    const int cc = min(SO_CC, ic - c0);
    float* tile = so_smem + buf * TILE;
    if (VEC) {
      for (int idx = threadIdx.x; idx < SO_CC * TH * G::CHUNKS; idx += SO_TX * SO_TY) {
        const int row = idx / G::CHUNKS, ch = idx - row * G::CHUNKS;
        const int c = row / TH, yy = row - c * TH, gy = y0 + yy - PAD, gx = x0 - 4 + 4 * ch;
        const bool ok = c < cc && gy >= 0 && gy < h && gx >= 0 && gx < wd;  // a chunk is wholly inside or wholly outside
        cp_async16_zfill(tile + row * TWP + 4 * ch, ok ? xs + (static_cast<long long>(c0 + c) * h + gy) * wd + gx : xs, ok);
      }
    } else
    for (int row = ty; row < SO_CC * TH; row += SO_TY) {  // one warp per tile row
      const int c = row / TH, yy = row - c * TH, gy = y0 + yy - PAD;
      const bool row_ok = c < cc && gy >= 0 && gy < h;
      const float* src = xs + (static_cast<long long>(c0 + c) * h + gy) * wd;
      float* dst = tile + row * TWP;
#pragma unroll
      for (int k = 0; k < NX; ++k) {
        if (xdst[k] < 0) continue;
        if (row_ok && xsrc[k] >= 0) cp_async4(dst + xdst[k], src + xsrc[k]);
        else dst[xdst[k]] = 0.0f;
      }
    }
    float* wch = so_smem + G::WOFF + buf * WCH;
    for (int i = threadIdx.x; i < OC * cc * KK; i += SO_TX * SO_TY) {
      const int o = i / (cc * KK), r = i - o * cc * KK;  // OIHW: (c, kh, kw) of the chunk are contiguous per o
      const int c = r / KK, t = r - c * KK, kh = t / KS, kw = t - kh * KS;
      cp_async4(wch + (c * KS + kh) * WROW + kw * OC + o, w + (static_cast<long long>(o) * ic + c0) * KK + r);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // SO_NBUF - 1 chunks in flight; one commit per iteration (an empty group past the end) keeps the wait count uniform
#pragma unroll
  for (int b = 0; b < SO_NBUF - 1; ++b) {
    if (b * SO_CC < ic) fetch(b * SO_CC, b);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  int cur = 0;
  for (int c0 = 0; c0 < ic; c0 += SO_CC, cur = cur + 1 == SO_NBUF ? 0 : cur + 1) {
    const int cc = min(SO_CC, ic - c0);
    asm volatile("cp.async.wait_group %0;" ::"n"(SO_NBUF - 2) : "memory");
    __syncthreads();  // this chunk has landed for every thread, and everyone is done with the buffer refilled next
    if (c0 + (SO_NBUF - 1) * SO_CC < ic) fetch(c0 + (SO_NBUF - 1) * SO_CC, cur == 0 ? SO_NBUF - 1 : cur - 1);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    const float* tile = so_smem + cur * TILE;
    const float* wch = so_smem + G::WOFF + cur * WCH;
    for (int c = 0; c < cc; ++c) {
#pragma unroll
      for (int r = 0; r < R + KS - 1; ++r) {  // input rows ascending = kernel rows ascending for every output row
        float seg[SEG];
        if (VEC) {
          // pixels x0 + 4 tx .. + 3 sit at tile columns 4 tx + 4 .. 4 tx + 7; the PAD values either side come from the neighbour
          // lanes' vectors (from shared memory at the two ends of the warp)
          const float* rowp = tile + (c * TH + ty * R + r) * TWP + 4 * tx;
          const float4 m = *reinterpret_cast<const float4*>(rowp + 4);
          const float mv[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
          for (int i = 0; i < SO_PX; ++i) seg[PAD + i] = mv[i];
#pragma unroll
          for (int i = 0; i < PAD; ++i) {
            const float lft = __shfl_up_sync(0xffffffffu, mv[SO_PX - PAD + i], 1);
            const float rgt = __shfl_down_sync(0xffffffffu, mv[i], 1);
            seg[i] = tx == 0 ? rowp[4 - PAD + i] : lft;
            seg[PAD + SO_PX + i] = tx == SO_TX - 1 ? rowp[8 + i] : rgt;
          }
        } else {
          const float* row = tile + (c * TH + ty * R + r) * TWP + tx * (SO_PX + 1);
#pragma unroll
          for (int i = 0; i < SEG; ++i) seg[i] = row[i + i / SO_PX];
        }
#pragma unroll
        for (int j = 0; j < R; ++j) {
          const int kh = r - j;
          if (kh < 0 || kh >= KS) continue;
          float wv[WROW];
          const float4* w4 = reinterpret_cast<const float4*>(wch + (c * KS + kh) * WROW);
#pragma unroll
          for (int v = 0; v < WROW / 4; ++v) {
            const float4 t = w4[v];
            wv[4 * v] = t.x, wv[4 * v + 1] = t.y, wv[4 * v + 2] = t.z, wv[4 * v + 3] = t.w;
          }
#pragma unroll
          for (int kw = 0; kw < KS; ++kw)
#pragma unroll
            for (int o = 0; o < OC; ++o)
#pragma unroll
              for (int q = 0; q < SO_PX; ++q) acc[o][j][q] = fmaf(seg[kw + q], wv[kw * OC + o], acc[o][j][q]);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < R; ++j) {
    const int gy = y0 + ty * R + j;
    if (gy >= h) continue;
#pragma unroll
    for (int o = 0; o < OC; ++o) {
#pragma unroll
      for (int q = 0; q < SO_PX; ++q) {
        const int gx = x0 + tx * SO_PX + q;
        if (gx < wd) {
          const long long oi = ((static_cast<long long>(n) * OC + o) * h + gy) * wd + gx;
          float v = acc[o][j][q];
          if (act == MIMIR_B200_ELT_RELU) v = fmaxf(v, 0.0f);
          else if (act == MIMIR_B200_ELT_SILU) v = v * (1.0f / (1.0f + expf(-v)));
          if (residual != nullptr) v += __ldg(residual + oi);
          y[oi] = v;
        }
      }
    }
  }
}

template <int OC, int KS, int VEC>
int launch_small_oc_v(const float* x, const float* w, float* y, const float* residual, int batch, int ic, int h, int wd, int act,
                      cudaStream_t st) {
  constexpr int R = so_rows(OC);
  using G = SmallOcGeom<KS, R, VEC>;
  constexpr int SMEM = (G::WOFF + SO_NBUF * SO_CC * KS * ((KS * OC + 3) & ~3)) * static_cast<int>(sizeof(float));
  static PerDeviceOnce attr_once;
  MB_TRY(attr_once.run([&]() -> int {
    MB_CUDA(cudaFuncSetAttribute(conv_small_oc_kernel<OC, KS, R, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    return MIMIR_B200_OK;
  }));
  dim3 grid((wd + SO_TX * SO_PX - 1) / (SO_TX * SO_PX), (h + SO_TY * R - 1) / (SO_TY * R), batch);
  conv_small_oc_kernel<OC, KS, R, VEC><<<grid, SO_TX * SO_TY, SMEM, st>>>(x, w, y, residual, ic, h, wd, act);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

template <int OC, int KS>
int launch_small_oc_k(const float* x, const float* w, float* y, const float* residual, int batch, int ic, int h, int wd, int act,
                      cudaStream_t st) {
  // whole 16-byte chunks per image row and an aligned base: the vector form (MIMIR_B200_CONV_SMALL_OC_VEC=0 turns it off)
  static const bool vec_off = [] { const char* e = getenv("MIMIR_B200_CONV_SMALL_OC_VEC"); return e && e[0] == '0'; }();
  if (!vec_off && (wd & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0)
    return launch_small_oc_v<OC, KS, 1>(x, w, y, residual, batch, ic, h, wd, act, st);
  return launch_small_oc_v<OC, KS, 0>(x, w, y, residual, batch, ic, h, wd, act, st);
}

template <int OC>
int launch_small_oc_t(const float* x, const float* w, float* y, const float* residual, int batch, int ic, int h, int wd, int ks, int pad,
                      int act, cudaStream_t st) {
  (void)pad;
  switch (ks) {
    case 1: return launch_small_oc_k<OC, 1>(x, w, y, residual, batch, ic, h, wd, act, st);
    case 3: return launch_small_oc_k<OC, 3>(x, w, y, residual, batch, ic, h, wd, act, st);
    case 5: return launch_small_oc_k<OC, 5>(x, w, y, residual, batch, ic, h, wd, act, st);
    case 7: return launch_small_oc_k<OC, 7>(x, w, y, residual, batch, ic, h, wd, act, st);
    default: return fail(MIMIR_B200_E_INVALID, "conv_small_oc: kernel size %d", ks);
  }
}

}  // namespace

bool conv_small_oc_supported(int oc, int ks, int stride, int pad, int h, int wd, int batch, int act) {
  static const bool off = [] { const char* e = getenv("MIMIR_B200_CONV_SMALL_OC"); return e && e[0] == '0'; }();
  return !off && oc >= 1 && oc <= SO_MAX_OC && stride == 1 && ks >= 1 && ks <= SO_MAX_KS && (ks & 1) == 1 && pad == ks / 2 && batch <= 65535 &&
         (h + SO_TY - 1) / SO_TY <= 65535 && (act == -1 || act == MIMIR_B200_ELT_RELU || act == MIMIR_B200_ELT_SILU) &&
         static_cast<long long>(h) * wd >= 4096;  // small images keep the tensor-core path (too few tiles to fill the SMs)
}

int launch_conv_small_oc(const float* x, const float* w, float* y, const float* residual, int batch, int ic, int oc, int h, int wd, int ks,
                         int pad, int act, cudaStream_t st) {
  switch (oc) {
    case 1: return launch_small_oc_t<1>(x, w, y, residual, batch, ic, h, wd, ks, pad, act, st);
    case 2: return launch_small_oc_t<2>(x, w, y, residual, batch, ic, h, wd, ks, pad, act, st);
    case 3: return launch_small_oc_t<3>(x, w, y, residual, batch, ic, h, wd, ks, pad, act, st);
    case 4: return launch_small_oc_t<4>(x, w, y, residual, batch, ic, h, wd, ks, pad, act, st);
    case 5: return launch_small_oc_t<5>(x, w, y, residual, batch, ic, h, wd, ks, pad, act, st);
    case 6: return launch_small_oc_t<6>(x, w, y, residual, batch, ic, h, wd, ks, pad, act, st);
    case 7: return launch_small_oc_t<7>(x, w, y, residual, batch, ic, h, wd, ks, pad, act, st);
    case 8: return launch_small_oc_t<8>(x, w, y, residual, batch, ic, h, wd, ks, pad, act, st);
    default: return fail(MIMIR_B200_E_INVALID, "conv_small_oc: %d output channels", oc);
  }
}

}  // namespace mb
