// attention_tc.cu — the attention core on the tensor cores (head_dim 64).
// Same arithmetic contract as attention.cu (LayerOps::self_attention_forward, LayerOps.hpp:1044-1090):
// s = (Q.K) / sqrt(hd), causal rows skip j > i, p = exp(s - max), p *= 1 / (sum p + 1e-9), O = P V.
//
// Flash-style with QK^T and PV on tcgen05 and the online softmax in registers:
//   * the operands are bf16 hi/lo planes.  Normally they are the planes [2][batch*seq][3E] that the QKV projection
//     GEMM writes from its epilogue, read in place through 5-D tensor maps (d, position, sample, head slot, plane):
//     Q and K tiles as [rows][64] (K-major for Q K^T), V tiles as [keys][64] rows used as an MN-major B operand of
//     P V - no pre-pass at all.  (From an fp32 QKV matrix, e.g. when a key / value cache is being filled, a pre-pass
//     lays the planes out per (sample, head), with V transposed to [64][seq] for a K-major P V.);
//   * one CTA owns 128 query rows of one (sample, head) and walks the keys in tiles of 64:
//       warp 0    TMA producer (Q once, then K_j, V_j; single-buffered, refilled as soon as the MMA
//                 that read them has completed)
//       warp 1    MMA issuer, one tile ahead on the scores: S_{j+1} = Q K_{j+1}^T (hi*hi + lo*hi + hi*lo)
//                 goes into the second of two TMEM score tiles while the softmax of tile j runs, then
//                 O += P_j V_j (same three products) accumulates in a third TMEM tile
//       warps 2-5 one thread per query row: tcgen05.ld S_j (the score tile is released as soon as it is
//                 in registers), running max / sum, P_j written to shared memory as bf16 hi/lo in the
//                 128-byte-swizzled K-major layout the MMA reads
//   * O stays in TMEM for the whole key loop.  The running maximum of a row is only raised when it grew
//     by more than 2^8 (decided per warp): then the warp waits for the last P V product, multiplies its
//     32 rows of O by exp(m_old - m_new) in place (tcgen05.ld / tcgen05.st) and carries on.  Otherwise
//     the stale maximum is kept - probabilities up to 2^8 are harmless in fp32 / split bf16 and the final
//     division by the row sum taken with the same maximum cancels it.  So there is no per-tile
//     read-modify-write of O and the softmax of tile j+1 overlaps P_j V_j.
//   * 96 KB of shared memory and 256 TMEM columns per CTA, so two CTAs share an SM.
// Every mbarrier wait is bounded; on expiry the CTA raises its abort flag, sets the device error word,
// leaves all loops and frees its TMEM.
#include "common.h"
#include "planes.cuh"
#include "sm100_ptx.cuh"

namespace mb {
namespace {

constexpr int AT_HD = 64;     // head dimension this kernel is written for
constexpr int AT_BQ = 128;    // query rows per CTA (TMEM lanes)
constexpr int AT_BK = 64;     // keys per tile
constexpr int AT_THREADS = 192;
constexpr int AT_TMEM_COLS = 256;  // two S tiles (64 each) + the O tile (64); a power of two

constexpr int AT_Q_BYTES = AT_BQ * AT_HD * 2;   // one plane
constexpr int AT_K_BYTES = 2 * AT_BK * AT_HD * 2;  // one plane of a PAIR of key tiles: Q K^T is issued for 128 keys at a time
constexpr int AT_V_BYTES = AT_HD * AT_BK * 2;
constexpr int AT_P_BYTES = AT_BQ * AT_BK * 2;
// no slack for aligning the base: two CTAs per SM leave none (the kernel checks the 1024-byte alignment it needs)
constexpr int AT_SMEM = 2 * AT_Q_BYTES + 2 * AT_K_BYTES + 2 * AT_V_BYTES + 2 * AT_P_BYTES + 256;

struct AttnParams {
  float* out;        // fp32 [batch*seq][embed], or nullptr
  __nv_bfloat16* out_split;  // or: bf16 hi (+ lo) operand planes [planes][batch*seq][embed] for the output projection
  long long plane_stride;
  int planes;
  int seq, embed, heads, causal;
  int bh;            // batch * heads
  float scale;
  int qk_from_planes;  // Q and K tiles come straight from the QKV GEMM's output planes [2][batch*seq][3E] (5-D maps)
  int v_mn_major;      // ... and so do the V tiles, as [key][d] rows read by the MMA as an MN-major B operand
  int f16;             // operand planes hold IEEE half instead of bfloat16
  int head_chunk;      // (sample, head) pairs per scheduling chunk of the second kernel form
  float acc_comp;      // relative loss of the truncating fp32 accumulation per MMA (0 = no compensation)
  int* err_word;
};

// fp32 QKV [batch*seq][3E] -> bf16 planes: Q, K as [plane][bh][seq][64]; V^T as [plane][bh][64][seqp]
__global__ void __launch_bounds__(256) attn_prep_kernel(const float* __restrict__ qkv, __nv_bfloat16* __restrict__ qp,
                                                        __nv_bfloat16* __restrict__ kp, __nv_bfloat16* __restrict__ vt, int seq,
                                                        int seqp, int embed, int heads, int bh, int f16) {
  __shared__ float tile[64][65];
  const int s0 = blockIdx.x * 64;       // 64 sequence positions
  const int b = blockIdx.y / heads, h = blockIdx.y - b * heads;
  const long long ld = 3LL * embed;
  const float* base = qkv + (static_cast<long long>(b) * seq) * ld + h * AT_HD;
  const long long qk_plane = static_cast<long long>(bh) * seq * AT_HD;
  const long long v_plane = static_cast<long long>(bh) * AT_HD * seqp;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // 64 x 4
  // Q and K: straight copies with the split
  for (int r = ty; r < 64; r += 4) {
    const int sidx = s0 + r;
    if (sidx < seq) {
      const float q = __ldg(base + sidx * ld + tx), k = __ldg(base + sidx * ld + embed + tx);
      const long long o = (static_cast<long long>(blockIdx.y) * seq + sidx) * AT_HD + tx;
      uint16_t qh, ql, kh, kl;
      split_one(q, f16, qh, ql);
      split_one(k, f16, kh, kl);
      reinterpret_cast<uint16_t*>(qp)[o] = qh;
      reinterpret_cast<uint16_t*>(qp)[o + qk_plane] = ql;
      reinterpret_cast<uint16_t*>(kp)[o] = kh;
      reinterpret_cast<uint16_t*>(kp)[o + qk_plane] = kl;
    }
    tile[r][tx] = (sidx < seq) ? __ldg(base + sidx * ld + 2 * embed + tx) : 0.0f;
  }
  __syncthreads();
  // V transposed: vt[bh][d][s]; positions past seq (up to seqp) are zero
  for (int d = ty; d < 64; d += 4) {
    const int sidx = s0 + tx;
    if (sidx < seqp) {
      const float v = tile[tx][d];
      const long long o = (static_cast<long long>(blockIdx.y) * AT_HD + d) * seqp + sidx;
      uint16_t vh, vl;
      split_one(v, f16, vh, vl);
      reinterpret_cast<uint16_t*>(vt)[o] = vh;
      reinterpret_cast<uint16_t*>(vt)[o + v_plane] = vl;
    }
  }
}

// V third of the QKV planes [2][batch*seq][3E] -> V^T planes [2][bh][64][seqp] (keys contiguous), zero past seq
__global__ void __launch_bounds__(256) attn_vt_kernel(const __nv_bfloat16* __restrict__ planes, __nv_bfloat16* __restrict__ vt, int seq,
                                                      int seqp, int embed, int heads, int bh, long long rows) {
  __shared__ __nv_bfloat16 tile[2][64][66];
  const int s0 = blockIdx.x * 64;
  const int b = blockIdx.y / heads, h = blockIdx.y - b * heads;
  const long long ld = 3LL * embed;
  const long long in_plane = rows * ld, v_plane = static_cast<long long>(bh) * AT_HD * seqp;
  const __nv_bfloat16* base = planes + (static_cast<long long>(b) * seq) * ld + 2 * embed + h * AT_HD;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const __nv_bfloat16 zero = __float2bfloat16_rn(0.0f);  // all-zero bits in either plane format
  for (int r = ty; r < 64; r += 4) {
    const int sidx = s0 + r;
    tile[0][r][tx] = (sidx < seq) ? base[sidx * ld + tx] : zero;
    tile[1][r][tx] = (sidx < seq) ? base[in_plane + sidx * ld + tx] : zero;
  }
  __syncthreads();
  for (int d = ty; d < 64; d += 4) {
    const int sidx = s0 + tx;
    if (sidx < seqp) {
      const long long o = (static_cast<long long>(blockIdx.y) * AT_HD + d) * seqp + sidx;
      vt[o] = tile[0][tx][d];
      vt[o + v_plane] = tile[1][tx][d];
    }
  }
}

__global__ void __launch_bounds__(AT_THREADS, 2)
flash_attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need it; never seen, but a wrong answer must not be silent
    if (threadIdx.x == 0) atomicExch(p.err_word, 29);
    return;
  }
  uint8_t* sQ = smem;                       // [2 planes][128][64] bf16, 128B-swizzled rows
  uint8_t* sK = sQ + 2 * AT_Q_BYTES;        // [2][128 keys][64]: two consecutive key tiles
  uint8_t* sV = sK + 2 * AT_K_BYTES;        // [2][64 d][64 keys]
  uint8_t* sP = sV + 2 * AT_V_BYTES;        // [2][128][64 keys]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * AT_P_BYTES);
  uint64_t *q_full = bars, *k_full = bars + 1, *k_empty = bars + 2, *v_full = bars + 3, *v_empty = bars + 4,
           *s_full = bars + 5 /* [2] */, *s_empty = bars + 7 /* [2] */, *p_full = bars + 9, *pv_done = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // causal: the query tiles with the most key tiles are scheduled first, so the last wave is made of short ones
  const int qt = p.causal ? static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
  const int bhi = blockIdx.y;
  const int q0 = qt * AT_BQ;
  int n_tiles = (p.seq + AT_BK - 1) / AT_BK;
  if (p.causal) n_tiles = min(n_tiles, (min(p.seq, q0 + AT_BQ) + AT_BK - 1) / AT_BK);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(s_full + 1, 1);
    mbar_init(s_empty, 4);
    mbar_init(s_empty + 1, 4);
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, AT_TMEM_COLS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 2 * AT_BK;  // score tile b lives at tmem_base + b * 64

  if (warp == 0) {
    if (lane == 0) {
      const int smp = bhi / p.heads, hd_slot = bhi - smp * p.heads;  // coordinates in the 5-D maps: (d, s, sample, head slot, plane)
      mbar_expect_tx(q_full, 2 * AT_Q_BYTES);
      if (p.qk_from_planes) {
        tma_load_5d(sQ, &map_q, q_full, 0, q0, smp, hd_slot, 0);
        tma_load_5d(sQ + AT_Q_BYTES, &map_q, q_full, 0, q0, smp, hd_slot, 1);
      } else {
        tma_load_3d(sQ, &map_q, q_full, 0, q0, bhi);
        tma_load_3d(sQ + AT_Q_BYTES, &map_q, q_full, 0, q0, p.bh + bhi);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const uint32_t ph = j & 1;
        if ((j & 1) == 0) {  // keys of tiles j and j + 1 in one 128-row box per plane
          const uint32_t pp = static_cast<uint32_t>(j >> 1) & 1;
          if (!mbar_wait(k_empty, pp ^ 1, abort_flag, p.err_word, 11)) break;
          mbar_expect_tx(k_full, 2 * AT_K_BYTES);
          if (p.qk_from_planes) {
            tma_load_5d(sK, &map_k, k_full, 0, j * AT_BK, smp, p.heads + hd_slot, 0);
            tma_load_5d(sK + AT_K_BYTES, &map_k, k_full, 0, j * AT_BK, smp, p.heads + hd_slot, 1);
          } else {
            tma_load_3d(sK, &map_k, k_full, 0, j * AT_BK, bhi);
            tma_load_3d(sK + AT_K_BYTES, &map_k, k_full, 0, j * AT_BK, p.bh + bhi);
          }
        }
        if (!mbar_wait(v_empty, ph ^ 1, abort_flag, p.err_word, 12)) break;
        mbar_expect_tx(v_full, 2 * AT_V_BYTES);
        if (p.v_mn_major) {
          tma_load_5d(sV, &map_v, v_full, 0, j * AT_BK, smp, 2 * p.heads + hd_slot, 0);
          tma_load_5d(sV + AT_V_BYTES, &map_v, v_full, 0, j * AT_BK, smp, 2 * p.heads + hd_slot, 1);
        } else {
          tma_load_3d(sV, &map_v, v_full, j * AT_BK, 0, bhi);
          tma_load_3d(sV + AT_V_BYTES, &map_v, v_full, j * AT_BK, 0, p.bh + bhi);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(AT_BQ, AT_BK, p.f16);  // M = 128, N = 64 for both products
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err_word, 13);
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP);
      // S for the key tiles 2 pr and 2 pr + 1 in one go: the two TMEM score tiles are adjacent, so Q [K_2pr ; K_2pr+1]^T is
      // a single N = 128 accumulator - twelve instructions for 128 keys instead of twenty-four (an instruction costs the
      // same tensor-pipe time at N = 64 and N = 128)
      const uint32_t idesc_s = make_idesc(AT_BQ, 2 * AT_BK, p.f16);
      auto issue_scores = [&](int pr) -> bool {
        const uint32_t u = static_cast<uint32_t>(pr) & 1;
        if (!mbar_wait(k_full, u, abort_flag, p.err_word, 14)) return false;
        if (!mbar_wait(s_empty, u ^ 1, abort_flag, p.err_word, 15)) return false;
        if (!mbar_wait(s_empty + 1, u ^ 1, abort_flag, p.err_word, 15)) return false;
        tcgen05_fence_after();
#pragma unroll
        for (int k = 0; k < AT_HD / 16; ++k) {
          const uint32_t ko = k * 32;
          const uint64_t qh = make_smem_desc(aQ + ko, 128), ql = make_smem_desc(aQ + AT_Q_BYTES + ko, 128);
          const uint64_t kh = make_smem_desc(aK + ko, 128), kl = make_smem_desc(aK + AT_K_BYTES + ko, 128);
          umma_bf16(tmem_base, qh, kh, idesc_s, k != 0 ? 1u : 0u);
          umma_bf16(tmem_base, ql, kh, idesc_s, 1u);
          umma_bf16(tmem_base, qh, kl, idesc_s, 1u);
        }
        umma_commit(s_full);
        umma_commit(s_full + 1);
        umma_commit(k_empty);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_scores(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const uint32_t ph = j & 1;
        if ((j & 1) == 1 && j + 1 < n_tiles && !issue_scores((j + 1) >> 1)) break;  // the next pair, once both score tiles are read
        if (!mbar_wait(p_full, ph, abort_flag, p.err_word, 16)) break;
        if (!mbar_wait(v_full, ph, abort_flag, p.err_word, 17)) break;
        tcgen05_fence_after();
#pragma unroll
        for (int k = 0; k < AT_BK / 16; ++k) {
          const uint32_t ko = k * 32;
          const uint64_t ph_ = make_smem_desc(aP + ko, 128), pl = make_smem_desc(aP + AT_P_BYTES + ko, 128);
          // V^T tile [d][keys]: K-major, 32 bytes along the row per 16 keys.  V tile [keys][d]: MN-major (bit 16 of the
          // instruction descriptor), one 128-byte row per key, so 16 keys are two 1024-byte groups of eight rows
          const uint32_t vo = p.v_mn_major ? k * 2048u : ko;
          const uint32_t id_pv = p.v_mn_major ? (idesc | (1u << 16)) : idesc;
          const uint64_t vh = make_smem_desc(aV + vo, 128), vl = make_smem_desc(aV + AT_V_BYTES + vo, 128);
          umma_bf16(tmem_o, ph_, vh, id_pv, (j != 0 || k != 0) ? 1u : 0u);
          umma_bf16(tmem_o, pl, vh, id_pv, 1u);
          umma_bf16(tmem_o, ph_, vl, id_pv, 1u);
        }
        umma_commit(pv_done);
        umma_commit(v_empty);
      }
    }
  } else {
    // ------------------------------ softmax: one thread per query row ------------------------------
    const int quad = warp & 3;
    const int r_local = quad * 32 + lane;
    const int row = q0 + r_local;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    constexpr float LOG2E = 1.4426950408889634f;
    float m_run = -1e30f, l_run = 0.0f;  // the reference's initial max (LayerOps.hpp:1052)
    uint8_t* p_row_hi = sP + r_local * 128;
    uint8_t* p_row_lo = p_row_hi + AT_P_BYTES;
    const int sw = r_local & 7;  // 128-byte swizzle: 16-byte chunk c of row r lives at chunk c ^ (r % 8)
    bool alive = true;
    // whole-warp wait: lane 0 runs the bounded wait, the others then see the completed phase at once
    auto warp_wait = [&](uint64_t* bar, uint32_t parity, int where) -> bool {
      int ok = 1;
      if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, p.err_word, where) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) return false;
      while (!mbar_try_wait(bar, parity)) {}
      return true;
    };
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j & 1;
      if (!warp_wait(s_full + b, static_cast<uint32_t>(j >> 1) & 1, 19)) { alive = false; break; }
      tcgen05_fence_after();
      const int key0 = j * AT_BK;
      // the whole tile of scores for this row, read once; the TMEM tile is free for S_{j+2} right away
      uint32_t sa[32], sb[32];
      const uint32_t tmem_s = tmem_base + b * AT_BK;
      tmem_ld_32x32_nowait(tmem_s + lane_base, sa);
      tmem_ld_32x32_nowait(tmem_s + lane_base + 32, sb);
      tmem_wait_ld();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty + b);
      // Tiles left of the diagonal and inside the sequence need no masking (warp-uniform test on the
      // warp's first row, which is the most restrictive one for the causal bound).
      const int row_first = q0 + quad * 32;
      const bool full_tile = (key0 + AT_BK <= p.seq) && (!p.causal || key0 + AT_BK - 1 <= row_first);
      const float c2 = p.scale * LOG2E;  // scores are kept in the exp2 domain: s * scale * log2(e)
      float mx = -1e30f;
      if (full_tile) {
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(sa[i]), __uint_as_float(sb[i])));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int ka = key0 + i, kb = key0 + 32 + i;
          if (!(ka < p.seq && (!p.causal || ka <= row))) sa[i] = 0xff800000u;  // -inf: contributes exp2(-inf) = 0
          if (!(kb < p.seq && (!p.causal || kb <= row))) sb[i] = 0xff800000u;
          mx = fmaxf(mx, fmaxf(__uint_as_float(sa[i]), __uint_as_float(sb[i])));
        }
      }
      // candidate maximum in score units (the reference's -1e30 start: LayerOps.hpp:1052)
      const float m_new = fmaxf(m_run, (mx > -1e30f) ? mx * p.scale : -1e30f);
      bool waited_pv = false;
      if (j == 0) {
        m_run = m_new;  // O is still empty: nothing to rescale
      } else {
        // raise the maximum only when some row of this warp outgrew it by more than 2^8
        const bool grow = (m_new - m_run) * LOG2E > 8.0f;
        if (__any_sync(0xffffffffu, grow)) {
          if (!warp_wait(pv_done, static_cast<uint32_t>(j - 1) & 1, 20)) { alive = false; break; }
          waited_pv = true;
          tcgen05_fence_after();
          const float corr = exp2f((m_run - m_new) * LOG2E);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t o[32];
            tmem_ld_32x32_nowait(tmem_o + lane_base + half * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
            tmem_st_32x32(tmem_o + lane_base + half * 32, o);
          }
          tmem_wait_st();
          l_run *= corr;
          m_run = m_new;
        }
      }
      const float m2 = m_run * LOG2E;
      // P_{j-1} V_{j-1} must have finished reading the P buffer before it is overwritten
      if (j > 0 && !waited_pv) {
        if (!warp_wait(pv_done, static_cast<uint32_t>(j - 1) & 1, 21)) { alive = false; break; }
      }
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {  // 16-byte chunks of 8 keys
          uint32_t hi[4], lo[4];
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            const uint32_t u0 = half ? sb[c8 * 8 + e] : sa[c8 * 8 + e];
            const uint32_t u1 = half ? sb[c8 * 8 + e + 1] : sa[c8 * 8 + e + 1];
            const float p0 = exp2f(fmaf(__uint_as_float(u0), c2, -m2));
            const float p1 = exp2f(fmaf(__uint_as_float(u1), c2, -m2));
            rs4[c8] += p0 + p1;
            split_pair(p0, p1, p.f16, hi[e >> 1], lo[e >> 1]);
          }
          const int chunk = (half * 4 + c8) ^ sw;
          *reinterpret_cast<uint4*>(p_row_hi + chunk * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          *reinterpret_cast<uint4*>(p_row_lo + chunk * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
      }
      l_run += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      // P is in shared memory and any rescaled O is back in TMEM: let the MMA warp issue P_j V_j
      tcgen05_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (alive && n_tiles > 0) alive = warp_wait(pv_done, static_cast<uint32_t>(n_tiles - 1) & 1, 22);
    if (alive) {
      tcgen05_fence_after();
      // 1 / (sum p + 1e-9) (LayerOps.hpp:1076), times the compensation for the truncating accumulation of P V: every
      // tcgen05.mma that added non-zero products into this row of O (three per 16 visible keys) lost about 1.5e-8 of
      // the running value (measured; the same constant as in the GEMM kernel).  Keys behind the causal mask add exact
      // zeros and lose nothing.
      const int keys_seen = p.causal ? min(p.seq, row + 1) : p.seq;
      const float inv = (1.0f + p.acc_comp * static_cast<float>(3 * ((keys_seen + 15) / 16))) / (l_run + 1e-9f);
      const int bb = bhi / p.heads, h = bhi - bb * p.heads;
      const long long o_off = (static_cast<long long>(bb) * p.seq + row) * p.embed + h * AT_HD;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t v[32];
        tmem_ld_32x32_nowait(tmem_o + lane_base + half * 32, v);  // every lane of the warp takes part in the load
        tmem_wait_ld();
        if (row < p.seq) {
          if (p.out != nullptr) {
            float* o = p.out + o_off;
#pragma unroll
            for (int c = 0; c < 32; c += 4)
              *reinterpret_cast<float4*>(o + half * 32 + c) =
                  make_float4(__uint_as_float(v[c]) * inv, __uint_as_float(v[c + 1]) * inv, __uint_as_float(v[c + 2]) * inv,
                              __uint_as_float(v[c + 3]) * inv);
          }
          if (p.out_split != nullptr) {
            __nv_bfloat16* oh = p.out_split + o_off + half * 32;
#pragma unroll
            for (int c = 0; c < 32; c += 8) {
              uint32_t hi[4], lo[4];
#pragma unroll
              for (int e = 0; e < 8; e += 2) {
                const float f0 = __uint_as_float(v[c + e]) * inv, f1 = __uint_as_float(v[c + e + 1]) * inv;
                split_pair(f0, f1, p.f16, hi[e >> 1], lo[e >> 1]);
              }
              *reinterpret_cast<uint4*>(oh + c) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
              if (p.planes == 2) *reinterpret_cast<uint4*>(oh + p.plane_stride + c) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
          }
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, AT_TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Second form of the kernel (the default when Q, K and V come from the projection's planes): the same arithmetic, a
// deeper pipeline.
//   * P never goes through shared memory.  The softmax threads write their probabilities back into tensor memory as
//     packed 16-bit pairs, over the columns of the score tile they were computed from (hi pairs in the first 32 columns
//     of the tile, lo pairs in the last 32), and P V is issued with its A operand in tensor memory.
//   * Three score tiles rotate (S_j -> P_j in tile j % 3), so the softmax of tile j + 1 starts as soon as S_{j+1} is
//     there; it no longer waits for P_j V_j to finish reading a single P buffer.  Q K^T runs two tiles ahead of P V.
//   * K and V tiles are double-buffered.
// Shared memory: Q 32 KB + 2 x 16 KB K + 2 x 16 KB V = 96 KB; 256 TMEM columns (3 x 64 scores + 64 for O): two CTAs
// per SM as before.  A tile's barriers live per score tile / per stage, so that no waiter is ever more than one phase
// behind the barrier it waits on.
constexpr int A2_TILE = AT_BK * AT_HD * 2;        // one plane of a 64-key K or V tile
constexpr int A2_STAGE = 2 * A2_TILE;             // hi and lo plane
constexpr int A2_THREADS = 320;                    // TMA warp, MMA warp, 8 softmax warps (two threads per query row)
constexpr int A2_XCHG = 4 * AT_BQ * 4;             // row maxima / sums exchanged between the two threads of a row
constexpr int A2_SMEM = 2 * AT_Q_BYTES + 2 * A2_STAGE + 2 * A2_STAGE + A2_XCHG + 256;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(A2_THREADS, 2)
flash_attn_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(p.err_word, 29);
    return;
  }
  uint8_t* sQ = smem;                       // [2 planes][128][64], 128B-swizzled rows
  uint8_t* sK = sQ + 2 * AT_Q_BYTES;        // [2 stages][2 planes][64 keys][64]
  uint8_t* sV = sK + 2 * A2_STAGE;          // [2 stages][2 planes][64 keys][64]
  float* xchg = reinterpret_cast<float*>(sV + 2 * A2_STAGE);  // [tile parity][key half][128 rows]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * A2_STAGE + A2_XCHG);
  uint64_t *q_full = bars, *k_full = bars + 1 /*[2]*/, *k_empty = bars + 3 /*[2]*/, *v_full = bars + 5 /*[2]*/, *v_empty = bars + 7 /*[2]*/,
           *s_full = bars + 9 /*[3]*/, *p_full = bars + 12 /*[3]*/, *pv_done = bars + 15 /*[3]*/;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* xchg_abort = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [4]: a warp of the pair gave up

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // CTA order.  Causal query tiles differ in length (2 ... 2 * q_tiles key tiles); within a chunk of `head_chunk`
  // (sample, head) pairs - sized so that the chunk's K and V stay in L2 - the longest tiles of all its heads are launched
  // first and the shortest last, so that the tail of the launch is made of short CTAs whatever the batch.
  int qt, bhi;
  {
    const int q_tiles = (p.seq + AT_BQ - 1) / AT_BQ;
    const int bid = static_cast<int>(blockIdx.x);
    const int c = bid / (q_tiles * p.head_chunk);
    const int rem = bid - c * q_tiles * p.head_chunk;
    const int hcnt = min(p.head_chunk, p.bh - c * p.head_chunk);
    const int rank = rem / hcnt;
    bhi = c * p.head_chunk + (rem - rank * hcnt);
    qt = p.causal ? q_tiles - 1 - rank : rank;
  }
  const int q0 = qt * AT_BQ;
  int n_tiles = (p.seq + AT_BK - 1) / AT_BK;
  if (p.causal) n_tiles = min(n_tiles, (min(p.seq, q0 + AT_BQ) + AT_BK - 1) / AT_BK);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full + i, 1);
      mbar_init(k_empty + i, 1);
      mbar_init(v_full + i, 1);
      mbar_init(v_empty + i, 1);
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(s_full + i, 1);
      mbar_init(p_full + i, 8);
      mbar_init(pv_done + i, 1);
    }
    *abort_flag = 0;
    for (int i = 0; i < 4; ++i) xchg_abort[i] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, AT_TMEM_COLS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 3 * AT_BK;  // score / probability tile b lives at tmem_base + b * 64

  if (warp == 0) {
    if (lane == 0) {
      const int smp = bhi / p.heads, hd_slot = bhi - smp * p.heads;  // 5-D maps: (d, position, sample, head slot, plane)
      mbar_expect_tx(q_full, 2 * AT_Q_BYTES);
      tma_load_5d(sQ, &map_q, q_full, 0, q0, smp, hd_slot, 0);
      tma_load_5d(sQ + AT_Q_BYTES, &map_q, q_full, 0, q0, smp, hd_slot, 1);
      bool ok = true;
      auto load_k = [&](int j) {
        const int st = j & 1;
        if (!mbar_wait(k_empty + st, (static_cast<uint32_t>(j >> 1) & 1) ^ 1, abort_flag, p.err_word, 31)) { ok = false; return; }
        mbar_expect_tx(k_full + st, A2_STAGE);
        tma_load_5d(sK + st * A2_STAGE, &map_k, k_full + st, 0, j * AT_BK, smp, p.heads + hd_slot, 0);
        tma_load_5d(sK + st * A2_STAGE + A2_TILE, &map_k, k_full + st, 0, j * AT_BK, smp, p.heads + hd_slot, 1);
      };
      auto load_v = [&](int j) {
        const int st = j & 1;
        if (!mbar_wait(v_empty + st, (static_cast<uint32_t>(j >> 1) & 1) ^ 1, abort_flag, p.err_word, 32)) { ok = false; return; }
        mbar_expect_tx(v_full + st, A2_STAGE);
        tma_load_5d(sV + st * A2_STAGE, &map_v, v_full + st, 0, j * AT_BK, smp, 2 * p.heads + hd_slot, 0);
        tma_load_5d(sV + st * A2_STAGE + A2_TILE, &map_v, v_full + st, 0, j * AT_BK, smp, 2 * p.heads + hd_slot, 1);
      };
      // in the order the MMA warp consumes them: K_0, K_1, then V_j, K_{j+2}
      if (n_tiles > 0) load_k(0);
      if (ok && n_tiles > 1) load_k(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        load_v(j);
        if (ok && j + 2 < n_tiles) load_k(j + 2);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(AT_BQ, AT_BK, p.f16);   // S = Q K^T: M = 128 queries, N = 64 keys
      const uint32_t idesc_pv = idesc_s | (1u << 16);             // O += P V: N = 64 (d), V rows are keys: MN-major B
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err_word, 33);
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
      auto issue_scores = [&](int j) -> bool {
        const uint32_t st = static_cast<uint32_t>(j) & 1, b = static_cast<uint32_t>(j % 3);
        if (!mbar_wait(k_full + st, static_cast<uint32_t>(j >> 1) & 1, abort_flag, p.err_word, 34)) return false;
        tcgen05_fence_after();
        const uint32_t kb = aK + st * A2_STAGE;
#pragma unroll
        for (int k = 0; k < AT_HD / 16; ++k) {
          const uint32_t ko = k * 32;
          const uint64_t qh = make_smem_desc(aQ + ko, 128), ql = make_smem_desc(aQ + AT_Q_BYTES + ko, 128);
          const uint64_t kh = make_smem_desc(kb + ko, 128), kl = make_smem_desc(kb + A2_TILE + ko, 128);
          umma_bf16(tmem_base + b * AT_BK, qh, kh, idesc_s, k != 0 ? 1u : 0u);
          umma_bf16(tmem_base + b * AT_BK, ql, kh, idesc_s, 1u);
          umma_bf16(tmem_base + b * AT_BK, qh, kl, idesc_s, 1u);
        }
        umma_commit(s_full + b);
        umma_commit(k_empty + st);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_scores(0);
      if (ok && n_tiles > 1) ok = issue_scores(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const uint32_t st = static_cast<uint32_t>(j) & 1, b = static_cast<uint32_t>(j % 3);
        if (!mbar_wait(p_full + b, static_cast<uint32_t>(j / 3) & 1, abort_flag, p.err_word, 35)) break;
        if (!mbar_wait(v_full + st, static_cast<uint32_t>(j >> 1) & 1, abort_flag, p.err_word, 36)) break;
        tcgen05_fence_after();
        const uint32_t tp = tmem_base + b * AT_BK;  // hi pairs in columns [0, 32), lo pairs in [32, 64) of the tile
        const uint32_t vb = aV + st * A2_STAGE;
#pragma unroll
        for (int k = 0; k < AT_BK / 16; ++k) {
          // 16 keys: eight packed columns of P, two 1024-byte groups of eight 128-byte V rows
          const uint64_t vh = make_smem_desc(vb + k * 2048u, 128), vl = make_smem_desc(vb + A2_TILE + k * 2048u, 128);
          umma_f16_ts(tmem_o, tp + k * 8, vh, idesc_pv, (j != 0 || k != 0) ? 1u : 0u);
          umma_f16_ts(tmem_o, tp + 32 + k * 8, vh, idesc_pv, 1u);
          umma_f16_ts(tmem_o, tp + k * 8, vl, idesc_pv, 1u);
        }
        umma_commit(pv_done + b);
        umma_commit(v_empty + st);
        if (j + 2 < n_tiles) {
          // S_{j+2} goes into the tile that P_{j-1} V_{j-1} read: that product has long finished (P_j came after it), the
          // wait only makes the reuse explicit
          if (j >= 1 && !mbar_wait(pv_done + (j - 1) % 3, static_cast<uint32_t>((j - 1) / 3) & 1, abort_flag, p.err_word, 37)) break;
          if (!issue_scores(j + 2)) break;
        }
      }
    }
  } else {
    // ------------------------------ softmax: two threads per query row ------------------------------
    // Warps 2-5 take the first 32 keys of every tile, warps 6-9 the last 32; the two warps that share a TMEM lane
    // quadrant (32 rows) agree on the row maxima through shared memory and a 64-thread named barrier per tile.
    const int quad = warp & 3;
    const int grp = (warp - 2) >> 2;  // which half of the tile's keys (and, at the end, of O's columns)
    const int r_local = quad * 32 + lane;
    const int row = q0 + r_local;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    constexpr float LOG2E = 1.4426950408889634f;
    float m_run = -1e30f, l_run = 0.0f;  // the reference's initial max (LayerOps.hpp:1052)
    bool alive = true;
    auto warp_wait = [&](uint64_t* bar, uint32_t parity, int where) -> bool {
      int ok = 1;
      if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, p.err_word, where) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) return false;
      while (!mbar_try_wait(bar, parity)) {}
      return true;
    };
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory"); };
    const float c2 = p.scale * LOG2E;  // scores are kept in the exp2 domain: s * scale * log2(e)
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j % 3;
      // a warp whose wait gave up keeps going round the loop without working, so that it meets its partner at every
      // pair barrier; the partner learns of it there and does the same (every wait returns at once while the abort flag is up)
      int ok_tile = 0;
      if (alive) ok_tile = warp_wait(s_full + b, static_cast<uint32_t>(j / 3) & 1, 38) ? 1 : 0;
      tcgen05_fence_after();
      const int key0 = j * AT_BK + grp * 32;
      uint32_t sc[32];
      const uint32_t tmem_s = tmem_base + b * AT_BK + lane_base;
      if (ok_tile) {
        tmem_ld_32x32_nowait(tmem_s + grp * 32, sc);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) sc[i] = 0u;
      }
      const int row_first = q0 + quad * 32;
      const bool full_tile = (key0 + 32 <= p.seq) && (!p.causal || key0 + 31 <= row_first);
      float mx = -1e30f;
      if (full_tile) {
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sc[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int ka = key0 + i;
          if (!(ka < p.seq && (!p.causal || ka <= row))) sc[i] = 0xff800000u;  // -inf: contributes exp2(-inf) = 0
          mx = fmaxf(mx, __uint_as_float(sc[i]));
        }
      }
      // the row's maximum over both halves of the tile (two exchange buffers: a thread may be one tile ahead of its partner)
      xchg[((j & 1) * 2 + grp) * AT_BQ + r_local] = mx;
      if (!ok_tile) xchg_abort[quad] = 1;
      pair_sync();
      if (xchg_abort[quad]) alive = false;
      if (!alive) continue;
      mx = fmaxf(mx, xchg[((j & 1) * 2 + (grp ^ 1)) * AT_BQ + r_local]);
      const float m_new = fmaxf(m_run, (mx > -1e30f) ? mx * p.scale : -1e30f);
      if (j == 0) {
        m_run = m_new;  // O is still empty: nothing to rescale
      } else {
        // raise the maximum only when some row of this quadrant outgrew it by more than 2^8 (both warps of the pair see
        // the same maxima, so they decide alike)
        const bool grow = (m_new - m_run) * LOG2E > 8.0f;
        if (__any_sync(0xffffffffu, grow)) {
          // every product issued so far has to be in O before it is rescaled; P_j V_j cannot start before both warps have
          // handed over their half of P_j, so O's rows are theirs alone until then (each warp its own 32 columns)
          if (!warp_wait(pv_done + (j - 1) % 3, static_cast<uint32_t>((j - 1) / 3) & 1, 39)) {
            alive = false;
            xchg_abort[quad] = 1;  // the partner sees it at the next pair barrier
            continue;
          }
          tcgen05_fence_after();
          const float corr = fast_exp2((m_run - m_new) * LOG2E);
          uint32_t o[32];
          tmem_ld_32x32_nowait(tmem_o + lane_base + grp * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
          tmem_st_32x32(tmem_o + lane_base + grp * 32, o);
          l_run *= corr;
          m_run = m_new;
        }
      }
      const float m2 = m_run * LOG2E;
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
      // probabilities of keys 2c, 2c + 1 become the packed pair in column c: hi pairs to columns [0, 32) of this score
      // tile, lo pairs to [32, 64) - the scores they replace are in registers already (this thread's and its partner's:
      // both loaded before the pair barrier above)
      uint32_t hi[16], lo[16];
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(sc[e]), c2, -m2));
        const float p1 = fast_exp2(fmaf(__uint_as_float(sc[e + 1]), c2, -m2));
        rs4[(e >> 1) & 3] += p0 + p1;
        split_pair(p0, p1, p.f16, hi[e >> 1], lo[e >> 1]);
      }
      tmem_st_32x16(tmem_s + grp * 16, hi);
      tmem_st_32x16(tmem_s + 32 + grp * 16, lo);
      l_run += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      // P (and any rescaled O) is in tensor memory: let the MMA warp issue P_j V_j
      tmem_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + b);
    }
    if (alive && n_tiles > 0) alive = warp_wait(pv_done + (n_tiles - 1) % 3, static_cast<uint32_t>((n_tiles - 1) / 3) & 1, 40);
    // the row sum over both halves (exchange buffer of the parity the last tile did not use)
    const int last = (n_tiles & 1) * 2;
    xchg[(last + grp) * AT_BQ + r_local] = l_run;
    if (!alive) xchg_abort[quad] = 1;
    pair_sync();
    if (xchg_abort[quad]) alive = false;
    if (alive) {
      l_run += xchg[(last + (grp ^ 1)) * AT_BQ + r_local];
      tcgen05_fence_after();
      const int keys_seen = p.causal ? min(p.seq, row + 1) : p.seq;
      const float inv = (1.0f + p.acc_comp * static_cast<float>(3 * ((keys_seen + 15) / 16))) / (l_run + 1e-9f);  // LayerOps.hpp:1076
      const int bb = bhi / p.heads, h = bhi - bb * p.heads;
      const long long o_off = (static_cast<long long>(bb) * p.seq + row) * p.embed + h * AT_HD + grp * 32;
      uint32_t v[32];
      tmem_ld_32x32_nowait(tmem_o + lane_base + grp * 32, v);  // every lane of the warp takes part in the load
      tmem_wait_ld();
      if (row < p.seq) {
        if (p.out != nullptr) {
          float* o = p.out + o_off;
#pragma unroll
          for (int c = 0; c < 32; c += 4)
            *reinterpret_cast<float4*>(o + c) = make_float4(__uint_as_float(v[c]) * inv, __uint_as_float(v[c + 1]) * inv,
                                                           __uint_as_float(v[c + 2]) * inv, __uint_as_float(v[c + 3]) * inv);
        }
        if (p.out_split != nullptr) {
          __nv_bfloat16* oh = p.out_split + o_off;
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint32_t h4[4], l4[4];
#pragma unroll
            for (int e = 0; e < 8; e += 2)
              split_pair(__uint_as_float(v[c + e]) * inv, __uint_as_float(v[c + e + 1]) * inv, p.f16, h4[e >> 1], l4[e >> 1]);
            *reinterpret_cast<uint4*>(oh + c) = make_uint4(h4[0], h4[1], h4[2], h4[3]);
            if (p.planes == 2) *reinterpret_cast<uint4*>(oh + p.plane_stride + c) = make_uint4(l4[0], l4[1], l4[2], l4[3]);
          }
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, AT_TMEM_COLS);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_map3(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t b0, uint32_t b1) {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  if (!fn) return fail(MIMIR_B200_E_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MIMIR_B200_E_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
  return MIMIR_B200_OK;
}

}  // namespace

bool attention_tc_supported(int seq, int embed, int heads) {
  const char* off = getenv("MIMIR_B200_ATTN_FP32");
  if (off && off[0] == '1') return false;
  return heads > 0 && embed == heads * AT_HD && seq >= 1;
}

size_t attention_tc_ws_bytes(int batch, int seq, int embed) {
  const size_t seqp = static_cast<size_t>(round_up(seq, 64));
  const size_t qk = 2ull * batch * seq * embed * 2;      // two planes of bf16
  const size_t v = 2ull * batch * embed * seqp * 2;
  return ((2 * qk + 255) & ~size_t(255)) + ((v + 255) & ~size_t(255)) + 512;
}

namespace {
// 5-D map over the QKV planes [2][batch*seq][3E]: (d in head, position, sample, head slot of Q|K|V, plane)
int make_map_qkv5(CUtensorMap* map, const void* base, int batch, int seq, int embed, uint32_t box_rows) {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  if (!fn) return fail(MIMIR_B200_E_CUDA, "cuTensorMapEncodeTiled entry point not available");
  const uint64_t ld = 3ull * embed;
  cuuint64_t dims[5] = {AT_HD, static_cast<cuuint64_t>(seq), static_cast<cuuint64_t>(batch), ld / AT_HD, 2};
  cuuint64_t strides[4] = {ld * 2, static_cast<cuuint64_t>(seq) * ld * 2, AT_HD * 2, static_cast<cuuint64_t>(batch) * seq * ld * 2};
  cuuint32_t box[5] = {AT_HD, box_rows, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MIMIR_B200_E_CUDA, "cuTensorMapEncodeTiled (QKV planes) failed (%d)", static_cast<int>(r));
  return MIMIR_B200_OK;
}

}  // namespace

int launch_attention_core_tc(const float* qkv, float* out, int batch, int seq, int embed, int heads, int causal, void* ws,
                             cudaStream_t st, __nv_bfloat16* out_split, int planes, const __nv_bfloat16* qkv_planes) {
  if (!attention_tc_supported(seq, embed, heads)) return fail(MIMIR_B200_E_UNSUPPORTED, "attention: tensor-core core needs head_dim 64");
  const int bh = batch * heads;
  const int seqp = round_up(seq, 64);
  if (bh > 65535 / 2) return fail(MIMIR_B200_E_UNSUPPORTED, "attention: batch * heads too large for one launch");
  uint8_t* w = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ws) + 255) & ~uintptr_t(255));
  const size_t qk_bytes = 2ull * batch * seq * embed * 2;
  __nv_bfloat16* qp = reinterpret_cast<__nv_bfloat16*>(w);
  __nv_bfloat16* kp = reinterpret_cast<__nv_bfloat16*>(w + qk_bytes);
  __nv_bfloat16* vt = reinterpret_cast<__nv_bfloat16*>(w + ((2 * qk_bytes + 255) & ~size_t(255)));
  dim3 pgrid(seqp / 64, bh);
  CUtensorMap mq, mk, mv;
  // (MIMIR_B200_ATTN_V_MN=0 goes back to the transposed V^T planes: decoder configuration 22.0 instead of 21.0 ms)
  static const bool v_mn_env = [] { const char* e = getenv("MIMIR_B200_ATTN_V_MN"); return !(e && e[0] == '0'); }();
  const bool v_mn = v_mn_env && qkv_planes != nullptr;
  // the deeper-pipelined form (P in tensor memory) takes the all-planes case; MIMIR_B200_ATTN_V2=0 keeps the first form
  static const bool v2_env = [] { const char* e = getenv("MIMIR_B200_ATTN_V2"); return !(e && e[0] == '0'); }();
  const bool v2 = v2_env && v_mn;
  if (qkv_planes != nullptr) {
    // Q and K are read where the projection GEMM left them; only V needs turning around
    if (!v_mn) {
      attn_vt_kernel<<<pgrid, 256, 0, st>>>(qkv_planes, vt, seq, seqp, embed, heads, bh, static_cast<long long>(batch) * seq);
      MB_CUDA(cudaGetLastError());
    }
    MB_TRY(make_map_qkv5(&mq, qkv_planes, batch, seq, embed, AT_BQ));
    MB_TRY(make_map_qkv5(&mk, qkv_planes, batch, seq, embed, v2 ? AT_BK : 2 * AT_BK));
  } else {
    attn_prep_kernel<<<pgrid, 256, 0, st>>>(qkv, qp, kp, vt, seq, seqp, embed, heads, bh, plane_format() == PLANES_F16);
    MB_CUDA(cudaGetLastError());
    MB_TRY(make_map3(&mq, qp, AT_HD, static_cast<uint64_t>(seq), 2ull * bh, AT_HD, AT_BQ));
    MB_TRY(make_map3(&mk, kp, AT_HD, static_cast<uint64_t>(seq), 2ull * bh, AT_HD, 2 * AT_BK));
  }
  if (v_mn) MB_TRY(make_map_qkv5(&mv, qkv_planes, batch, seq, embed, AT_BK));
  else MB_TRY(make_map3(&mv, vt, static_cast<uint64_t>(seqp), AT_HD, 2ull * bh, AT_BK, AT_HD));
  static PerDeviceOnce attr_once;
  MB_TRY(attr_once.run([&]() -> int {
    MB_CUDA(cudaFuncSetAttribute(flash_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM));
    return MIMIR_B200_OK;
  }));
  AttnParams p;
  p.out = out;
  p.out_split = out_split;  // embed = heads * 64, so the planes' padded row length equals embed
  p.plane_stride = static_cast<long long>(batch) * seq * embed;
  p.planes = planes;
  p.qk_from_planes = qkv_planes != nullptr ? 1 : 0;
  p.v_mn_major = v_mn ? 1 : 0;
  p.seq = seq; p.embed = embed; p.heads = heads; p.causal = causal; p.bh = bh;
  p.scale = 1.0f / sqrtf(static_cast<float>(AT_HD));
  p.err_word = ctx().dev_error_word;
  static const bool comp = [] { const char* e = getenv("MIMIR_B200_ACC_COMP"); return !(e && e[0] == '0'); }();
  p.acc_comp = comp ? 1.5e-8f : 0.0f;
  p.f16 = plane_format() == PLANES_F16 ? 1 : 0;
  dim3 grid((seq + AT_BQ - 1) / AT_BQ, bh);
  p.head_chunk = 1;
  if (v2) {
    // heads whose K and V planes (seq x 64 x 2 planes x 2 bytes, twice) fill about 48 MB of L2
    const long long per_head = static_cast<long long>(seq) * AT_HD * 2 * 2 * 2;
    long long hc = (48ll << 20) / per_head;
    p.head_chunk = static_cast<int>(hc < 1 ? 1 : (hc > bh ? bh : hc));
    grid = dim3(static_cast<unsigned>(((seq + AT_BQ - 1) / AT_BQ) * bh));
    static PerDeviceOnce attr2_once;
    MB_TRY(attr2_once.run([&]() -> int {
      MB_CUDA(cudaFuncSetAttribute(flash_attn_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A2_SMEM));
      return MIMIR_B200_OK;
    }));
    flash_attn_tc2_kernel<<<grid, A2_THREADS, A2_SMEM, st>>>(mq, mk, mv, p);
    MB_CUDA(cudaGetLastError());
    count_launch(1);
    return MIMIR_B200_OK;
  }
  flash_attn_tc_kernel<<<grid, AT_THREADS, AT_SMEM, st>>>(mq, mk, mv, p);
  MB_CUDA(cudaGetLastError());
  count_launch(2);
  return MIMIR_B200_OK;
}

}  // namespace mb
