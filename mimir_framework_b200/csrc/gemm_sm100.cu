// gemm_sm100.cu — the contraction kernel every dense layer funnels into (Linear, the attention
// projections, Conv2d lowered to GEMM).  Replaces LayerOps::linear_forward (LayerOps.hpp:24-111)
// and HardwareOpt::matmul_fma_saturated (HardwareOpt.hpp:95-149).
//
//   Y[m, n] = act( sum_k A[m, k] * W[n, k] + bias[n] ) (+ residual[m, n])
//
// Both operands are K-major ("TN"), which is the reference's Linear layout (W is [out][in]).
// fp32 operands are carried as bf16 planes: x = hi + lo with hi = bf16(x), lo = bf16(x - hi).
// The kernel issues hi*hi + lo*hi + hi*lo (the lo*lo term, ~2^-18 relative, is dropped) with fp32
// accumulation in tensor memory, which keeps the result within ~2^-16 per product of the fp32
// CPU path while running on the bf16 tensor pipe.
//
// sm_100a structure (one CTA per SM, persistent over output tiles):
//   warp 0      : TMA producer  — cp.async.bulk.tensor (no multicast) into a ring of smem stages
//   warp 1      : MMA issuer    — one thread issues tcgen05.mma, operands from smem descriptors,
//                                 accumulators in TMEM (2 x 256 columns, double buffered)
//   warps 2..9  : epilogue      — tcgen05.ld TMEM -> registers, bias / activation / residual, 256-bit
//                                 stores of fp32 rows and/or the bf16 hi/lo planes of the next layer
//                                 (or channel-major NCHW for convs)
// Every mbarrier wait is bounded: after ~2 s it sets the device error word and the CTA drains.
#include "common.h"
#include "planes.cuh"
#include "sm100_ptx.cuh"

#include <cmath>
#include <cstring>

namespace mb {

namespace {

constexpr int BM = 128;        // rows of the output tile (TMEM lanes)
constexpr int BN = 256;        // columns of the output tile (one MMA, N = 256)
constexpr int UMMA_K = 16;     // bf16 K per tcgen05.mma
constexpr int NUM_ACC = 2;     // TMEM accumulator buffers
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 320;  // 10 warps: TMA, MMA, 8 epilogue
constexpr int EPI_WARPS = 8;
constexpr float ACC_TRUNC_PER_MMA = 1.5e-8f;  // mean relative loss of the fp32 accumulator per tcgen05.mma (truncating adds)

// GELU in the reference's tanh form (LayerOps.hpp:556-568), x * 0.5 * (1 + tanh(u)) with u = c * (x + 0.044715 x^3) and
// c = sqrt(2.0f / 3.14159265359f) evaluated in fp32.  0.5 * (1 + tanh(u)) is the logistic function of 2u, so the value is
// x / (1 + exp(-2u)): one ex2 and one reciprocal on the special-function unit instead of tanhf's ~30 instructions (the
// epilogue of a K = 768 layer has only ~12 000 cycles per 128 x 256 tile for 32 768 of these), and without the
// cancellation of 1 + tanh(u) for negative arguments.  Error: a few ulp of the result (ex2.approx 2 ulp, rcp.approx 1 ulp).
__device__ __forceinline__ float gelu_ref(float x) {
  const float c = 0.7978845608f;
  const float u = c * (x + 0.044715f * x * x * x);
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(u * -2.885390082f));  // exp(-2u) = 2^(-2u log2 e)
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}
__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case MIMIR_B200_ELT_GELU: return gelu_ref(v);
    case MIMIR_B200_ELT_SILU: return v * (1.0f / (1.0f + expf(-v)));
    case MIMIR_B200_ELT_RELU: return fmaxf(v, 0.0f);
    case MIMIR_B200_ELT_TANH: return tanhf(v);
    case MIMIR_B200_ELT_SIGMOID: return 1.0f / (1.0f + expf(-v));
    default: return v;
  }
}

struct GemmParams {
  int m, n, kblocks;         // kblocks = kp / BK
  int a_planes, w_planes;
  int tiles_m, tiles_n, group_n;
  const float* bias;
  const float* residual;
  int activation;
  float* out_f32;
  long long ldo;
  __nv_bfloat16* out_split;  // [2][m][np]
  long long np;              // round_up(n, 64)
  int ohw;                   // > 0: fp32 output (and residual) are NCHW, row = sample * ohw + pixel
  int bn;                    // columns of an output tile = N of one MMA: BN, or 192 on request (plain row-major form only)
  // Convolution as a sum of shifted GEMMs (conv_ks > 0): A is the zero-padded NHWC activation matrix
  // [samples * hp * wp, C]; k-block kb belongs to tap t = kb / conv_cblocks and reads A rows shifted by
  // (kh - pad) * wp + (kw - pad); output rows live on the padded grid, border rows are dropped.
  int conv_ks, conv_cblocks, conv_pad, conv_hp, conv_wp, conv_h, conv_w;
  // swap != 0 (channel-major outputs with at most 128 output channels): the weights are the M side of the
  // MMA (TMEM lane = output channel) and 256 activation rows are its N side.  A tcgen05.mma with M = 128 costs
  // the same whatever its N, so a narrow layer computed the usual way (N = its few channels, padded to the
  // tile) pays for 256 columns it does not have; swapped, every instruction does full work.
  int swap;
  int tma_store;  // fp32 row-major output leaves through TMA stores (map_o) instead of per-lane stores
  // Every accumulator is multiplied by this before bias / activation: 1 + ACC_TRUNC_PER_MMA * (MMAs per output).
  // The tensor core adds each MMA's products to the fp32 accumulator with truncation, not round-to-nearest, which
  // shrinks every result by a little less than 2^-26 of its value per instruction (see launch_gemm_t).
  float acc_scale;
  int f16;        // operand planes (and out_split) hold IEEE half instead of bfloat16
  // The operand ring: a stage holds only the planes the precision mode uses (32 KB with two activation planes and one
  // weight plane at BK = 32), so the same shared memory gives six stages instead of four - the K = 768 layers were
  // starved of operands with four (the MMA thread spent a quarter of every tile waiting on a full barrier).
  int stages, stage_bytes;
  int* err_word;
  // grouped form: W rows of tile (tm, tn) start at (tm * BM / a_group_rows) * w_group_rows + tn * bn (0 = one group)
  int a_group_rows, w_group_rows;
  // Channel-major forms: per-(32-pixel block, 32-channel chunk) GroupNorm partials of the values stored, for the GroupNorm that
  // reads this output (gn_part != null): entry [block * chunks + chunk][set][pixels, (sum, sum of squares) per group],
  // set 0 = the sample of the block's first row, set 1 = the next sample where a block straddles two.
  float* gn_part;
  int gn_cpg;  // channels per group (4, 8, 16 or 32)
};

// Tile order: groups of `group_n` column tiles; inside a group the row tile runs fastest, so the
// CTAs resident at one time share a few W column tiles (kept in L2) while A streams through.
__device__ __forceinline__ void tile_coords(int t, const GemmParams& p, int& tm, int& tn) {
  const int per_group = p.group_n * p.tiles_m;
  const int g = t / per_group;
  const int r = t - g * per_group;
  const int gn0 = g * p.group_n;
  const int gw = min(p.group_n, p.tiles_n - gn0);
  tn = gn0 + r % gw;
  tm = r / gw;
}

template <int BK>
struct SmemLayout {
  static constexpr int kATile = BM * BK * 2;
  static constexpr int kWTile = BN * BK * 2;
};

constexpr int MAX_STAGES = 8;

// GroupNorm partials of one 32-pixel x 32-channel chunk (a lane = a pixel, v = its 32 channels as stored): per group of CPG
// channels the sum and the sum of squares over the lanes of the set, plus the set's pixel count.  The 2 * (32 / CPG) per-lane
// values meet by recursive halving (a lane hands over half of what it holds per round: 2G - 1 shuffles, not 5 per value), the
// lanes that end up with a total store it.  Entry of a set: [pixels, S_0, Q_0, S_1, Q_1, ...].
template <int CPG>
__device__ __forceinline__ void gn_emit_set(const float (&v)[32], bool in, int nvalid_ch, int lane, float* dst) {
  constexpr int G = 32 / CPG, G2 = 2 * G;
  float a[G2];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float s = 0.0f, q = 0.0f;
#pragma unroll
    for (int j = 0; j < CPG; ++j)
      if (in && g * CPG + j < nvalid_ch) { s += v[g * CPG + j]; q = fmaf(v[g * CPG + j], v[g * CPG + j], q); }
    a[2 * g] = s;
    a[2 * g + 1] = q;
  }
  int mask = 16;
#pragma unroll
  for (int half = G2 / 2; half >= 1; half >>= 1, mask >>= 1) {
    const bool upper = (lane & mask) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float send = upper ? a[i] : a[i + half];
      const float keep = upper ? a[i + half] : a[i];
      a[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
    }
  }
  for (; mask >= 1; mask >>= 1) a[0] += __shfl_xor_sync(0xffffffffu, a[0], mask);  // the lanes that hold the same value index
  const unsigned bal = __ballot_sync(0xffffffffu, in);
  if (lane == 0) dst[0] = static_cast<float>(__popc(bal));
  if ((lane & (32 / G2 - 1)) == 0) dst[1 + lane / (32 / G2)] = a[0];
}
// smp: the sample of this lane's row (rows past the matrix included: row / per); row_in: the row exists; pix_ok: it is a stored pixel
__device__ __forceinline__ void gn_emit_chunk(const float (&v)[32], bool pix_ok, bool row_in, int smp, int nvalid_ch, int lane, int cpg,
                                              float* dst) {
  const int smp0 = __shfl_sync(0xffffffffu, smp, 0);
  const bool next = __any_sync(0xffffffffu, row_in && smp != smp0);
  const int es = 1 + 64 / cpg;  // floats per set
  for (int set = 0; set < (next ? 2 : 1); ++set) {
    const bool in = pix_ok && smp == smp0 + set;
    float* d = dst + set * es;
    switch (cpg) {
      case 4: gn_emit_set<4>(v, in, nvalid_ch, lane, d); break;
      case 8: gn_emit_set<8>(v, in, nvalid_ch, lane, d); break;
      case 16: gn_emit_set<16>(v, in, nvalid_ch, lane, d); break;
      default: gn_emit_set<32>(v, in, nvalid_ch, lane, d); break;
    }
  }
}

// CM = 1 compiles the channel-major forms in (NCHW output, convolution as shifted GEMMs, swapped operands; CM = 2: the same
// plus GroupNorm partials of the stored values from the epilogue); the plain
// row-major form (CM = 0: every Linear and attention projection) is built without them, so that the two families
// neither share a register budget nor slow each other's epilogue down.
// PAIR = 1 (not with swapped operands): the kernel runs as clusters of two CTAs on neighbouring SMs that share one 256-row x 256-column
// tile (tcgen05 with cta_group::2).  Each CTA loads its own 128 rows of A and only HALF of the W tile; the even-ranked
// CTA issues the MMAs for both, each CTA reads its 128 accumulator rows out of its own tensor memory.  The operand
// bytes an SM pulls from L2 per MMA cycle drop by a quarter to a third, which is what the short-K layers are short of.
template <int BK, int RING_BYTES, int CM, int PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tn_bf16split_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ CUtensorMap map_o, const GemmParams p) {
  constexpr int SWZ = BK * 2;                      // bytes per smem row = swizzle span
  constexpr int A_TILE = BM * BK * 2;
  constexpr int W_TILE = (PAIR ? BN / 2 : BN) * BK * 2;  // a CTA of a pair holds half of the N side
  const int STAGES = p.stages, STAGE_BYTES = p.stage_bytes;
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;  // 0 = the pair's leader
  const int t_first = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int t_step = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // behind the stages: one staging tile per epilogue warp (32 x 33 floats for the swapped form's transposition, or a
  // dense 128-byte-swizzled 32 x 32 tile, 1024-byte aligned, as the source of a TMA store), then the barriers
  uint8_t* epi_tiles = smem + RING_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_tiles + EPI_WARPS * 32 * 33 * 4);
  uint64_t* empty_bar = full_bar + MAX_STAGES;
  uint64_t* acc_full = empty_bar + MAX_STAGES;
  uint64_t* acc_empty = acc_full + NUM_ACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + NUM_ACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], PAIR ? 2 * EPI_WARPS : EPI_WARPS);  // the leader's collects both CTAs' epilogue warps
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_slot, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // planes on the M side (128-row tiles) and on the N side (256-row tiles) of the MMA
  const bool swapped = CM && p.swap;
  const bool conv = CM && p.conv_ks > 0;
  const int m_planes = swapped ? p.w_planes : p.a_planes, n_planes = swapped ? p.a_planes : p.w_planes;
  const uint32_t tx_bytes = PAIR ? static_cast<uint32_t>(2 * (m_planes * A_TILE + n_planes * W_TILE))  // both CTAs' loads land on the leader's barrier
                                 : static_cast<uint32_t>(m_planes * A_TILE + n_planes * (p.bn * BK * 2));

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = t_first; t < num_tiles && ok; t += t_step) {
        int tm, tn;
        tile_coords(t, p, tm, tn);
        if (PAIR) tm = tm * 2 + static_cast<int>(crank);  // p.tiles_m counts row PAIRS
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err_word, 1)) { ok = false; break; }
          uint8_t* sbase = smem + stage * STAGE_BYTES;
          int a_col = kb * BK, a_row = tm * BM;
          if (conv) {
            const int t = kb / p.conv_cblocks, cb = kb - t * p.conv_cblocks;
            const int kh = t / p.conv_ks, kw = t - kh * p.conv_ks;
            a_row += (kh - p.conv_pad) * p.conv_wp + (kw - p.conv_pad);  // may be negative: TMA zero-fills
            a_col = cb * BK;
          }
          if (PAIR) {
            // the leader arms its barrier for the bytes of both CTAs; this CTA's bytes are counted there whichever
            // of the two arrives first (the phase cannot complete before the leader's arrive)
            if (crank == 0) mbar_expect_tx(&full_bar[stage], tx_bytes);
            const uint32_t fb = mapa_shared(smem_u32(&full_bar[stage]), 0);
            for (int pl = 0; pl < p.a_planes; ++pl)
              tma_load_3d_pair(sbase + pl * A_TILE, &map_a, fb, a_col, a_row, pl);
            for (int pl = 0; pl < p.w_planes; ++pl)
              tma_load_3d_pair(sbase + m_planes * A_TILE + pl * W_TILE, &map_w, fb, kb * BK, tn * BN + static_cast<int>(crank) * (BN / 2), pl);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
            continue;
          }
          mbar_expect_tx(&full_bar[stage], tx_bytes);
          if (!swapped) {
            for (int pl = 0; pl < p.a_planes; ++pl)
              tma_load_3d(sbase + pl * A_TILE, &map_a, &full_bar[stage], a_col, a_row, pl);
            for (int pl = 0; pl < p.w_planes; ++pl)
              tma_load_3d(sbase + m_planes * A_TILE + pl * W_TILE, &map_w, &full_bar[stage], kb * BK,
                          tn * p.bn + (p.a_group_rows > 0 ? (tm * BM / p.a_group_rows) * p.w_group_rows : 0), pl);
          } else {
            // 128 weight rows into the M-side tiles, 256 activation rows (tile tn) into the N-side tiles
            a_row += tn * BN - tm * BM;
            for (int pl = 0; pl < p.w_planes; ++pl)
              tma_load_3d(sbase + pl * A_TILE, &map_w, &full_bar[stage], kb * BK, tm * BM, pl);
            for (int pl = 0; pl < p.a_planes; ++pl)
              tma_load_3d(sbase + m_planes * A_TILE + pl * W_TILE, &map_a, &full_bar[stage], a_col, a_row, pl);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // Drain: every stage this thread filled must have landed and been consumed (or the abort
      // flag is up) before the CTA may exit with copies in flight.
      for (int s = 0; s < STAGES; ++s) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err_word, 2)) break;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------------------
    if (lane == 0 && crank == 0) {
      const uint32_t idesc = make_idesc(PAIR ? 2 * BM : BM, p.bn, p.f16);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = t_first; t < num_tiles && ok; t += t_step) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.err_word, 3)) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.err_word, 4)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sw = sa + m_planes * A_TILE;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t koff = k * UMMA_K * 2;  // bytes along K inside the swizzled row
            const uint64_t a_hi = make_smem_desc(sa + koff, SWZ);
            const uint64_t w_hi = make_smem_desc(sw + koff, SWZ);
            if (PAIR) umma_bf16_pair(d_tmem, a_hi, w_hi, idesc, (kb | k) != 0 ? 1u : 0u);
            else umma_bf16(d_tmem, a_hi, w_hi, idesc, (kb | k) != 0 ? 1u : 0u);
            if (m_planes == 2) {
              const uint64_t a_lo = make_smem_desc(sa + A_TILE + koff, SWZ);
              if (PAIR) umma_bf16_pair(d_tmem, a_lo, w_hi, idesc, 1u);
              else umma_bf16(d_tmem, a_lo, w_hi, idesc, 1u);
            }
            if (n_planes == 2) {
              const uint64_t w_lo = make_smem_desc(sw + W_TILE + koff, SWZ);
              if (PAIR) umma_bf16_pair(d_tmem, a_hi, w_lo, idesc, 1u);
              else umma_bf16(d_tmem, a_hi, w_lo, idesc, 1u);
            }
          }
          if (PAIR) {  // frees the stage in both CTAs when these MMAs have read it
            umma_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 0));
            umma_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 1));
          } else
          umma_commit(&empty_bar[stage]);  // frees the stage when these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (PAIR) {
          umma_commit_pair(mapa_shared(smem_u32(&acc_full[acc]), 0));
          umma_commit_pair(mapa_shared(smem_u32(&acc_full[acc]), 1));
        } else
        umma_commit(&acc_full[acc]);
        if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..9) ---------------------------------
    // Two warps per TMEM lane quadrant, each owning half of the tile's columns.  A lane holds 32 consecutive
    // columns of its row: row-major outputs leave as whole 128-byte lines through 256-bit stores;
    // channel-major (NCHW) outputs are coalesced across lanes (lane <-> pixel).
    const int ew = warp - 2;
    const int quad = warp & 3;   // TMEM lane quadrant this warp may read
    const int half = ew >> 2;    // which half of the columns
    const bool chan_major = CM && (p.ohw > 0 || p.conv_ks > 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = t_first; t < num_tiles; t += t_step) {
      int tm, tn;
      tile_coords(t, p, tm, tn);
      if (PAIR) tm = tm * 2 + static_cast<int>(crank);
      // lane 0 does the bounded wait; the verdict is made warp-uniform because tcgen05.ld below
      // is a warp-collective instruction
      int ok = 1;
      if (lane == 0) ok = mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.err_word, 5) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      while (!mbar_try_wait(&acc_full[acc], acc_phase)) {}  // completes at once: lane 0 saw the phase
      tcgen05_fence_after();
      const int row0 = tm * BM + quad * 32;
      const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * BN);
      if (swapped) {
        // TMEM lane = output channel, column = activation row (pixel).  Each 32 x 32 chunk is turned around
        // through a padded shared-memory tile so that a lane owns a pixel again and the NCHW stores (and
        // residual loads) of a warp are 128 contiguous bytes per channel, as in the unswapped form.
        float* tbuf = reinterpret_cast<float*>(epi_tiles) + ew * (32 * 33);
        const int oc0 = row0;  // first output channel of this warp's 32 lanes
        const long long hw = conv ? static_cast<long long>(p.conv_h) * p.conv_w : static_cast<long long>(p.ohw);
        // where this lane's pixel of chunk ci lands in the NCHW output; false = the chunk is past the matrix (warp-uniform)
        int g_smp = 0;       // sample of this lane's row in the chunk geom() was last asked about
        bool g_row_in = false;
        auto geom = [&](int ci, int& c0, bool& pv, long long& o0) -> bool {
          c0 = (half * (BN / 64) + ci) * 32;
          const int r0 = tn * BN + c0;
          if (r0 >= p.m || oc0 >= p.n) return false;
          const int prow = r0 + lane;
          pv = prow < p.m;
          g_row_in = pv;
          long long pbase = 0;
          if (conv) {
            const int per = p.conv_hp * p.conv_wp;
            const int smp = prow / per, rem = prow - smp * per;
            g_smp = smp;
            const int yq = rem / p.conv_wp;
            const int yy = yq - p.conv_pad, xx = rem - yq * p.conv_wp - p.conv_pad;
            pv = pv && yy >= 0 && yy < p.conv_h && xx >= 0 && xx < p.conv_w;
            pbase = static_cast<long long>(smp) * p.n * hw + static_cast<long long>(yy) * p.conv_w + xx;
          } else {
            const long long smp = prow / p.ohw;
            g_smp = static_cast<int>(smp);
            pbase = smp * p.n * hw + (prow - smp * p.ohw);
          }
          o0 = pbase + static_cast<long long>(oc0) * hw;
          return true;
        };
        const bool full = oc0 + 32 <= p.n;
        // With a short K the epilogue, not the MMA, sets the pace.  The residual of a chunk is requested before the chunk
        // is read out of tensor memory and turned around, and the lines of the next chunk are pulled into L2 meanwhile, so
        // that the loads do not each wait a full memory latency.
        constexpr int NCH = (BN / 32) / 2;
#pragma unroll 1
        for (int ci = 0; ci < NCH; ++ci) {
          int c0; bool pv; long long o0;
          if (!geom(ci, c0, pv, o0)) break;
          const int my_smp = g_smp;
          const bool my_row_in = g_row_in;
          float q[32];
          if (p.residual != nullptr) {
            if (pv) {
#pragma unroll
              for (int j = 0; j < 32; ++j) q[j] = (full || oc0 + j < p.n) ? __ldg(p.residual + o0 + j * hw) : 0.0f;
            }
            int c1; bool pv1; long long o1;
            if (ci + 1 < NCH && geom(ci + 1, c1, pv1, o1) && pv1) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (full || oc0 + j < p.n) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.residual + o1 + j * hw));
            }
          }
          float v[32];
          tmem_ld_32x32(taddr0 + c0, v);
#pragma unroll
          for (int j = 0; j < 32; ++j) tbuf[j * 33 + lane] = v[j] * p.acc_scale;  // [pixel][channel]
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = tbuf[lane * 33 + j];  // lane = pixel r0 + lane, j = channel oc0 + j
          __syncwarp();
          if (p.activation != -1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.activation);
          }
          if (pv) {
            if (p.residual != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += q[j];
            }
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || oc0 + j < p.n) p.out_f32[o0 + j * hw] = v[j];
          }
          if (CM == 2 && p.gn_part != nullptr) {
            const long long blk = (tn * BN + c0) >> 5;
            float* gd = p.gn_part + (blk * ((p.n + 31) >> 5) + (oc0 >> 5)) * (2 * (1 + 64 / p.gn_cpg));
            gn_emit_chunk(v, pv, my_row_in, my_smp, min(32, p.n - oc0), lane, p.gn_cpg, gd);
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1; }
        continue;
      }
      const int col_limit = (p.out_split != nullptr) ? static_cast<int>(p.np) : p.n;
      // channel-major addressing of this lane's row
      bool cm_ok = false, cm_row_in = false;
      int cm_smp = 0;
      long long cm_o0 = 0, cm_stride = 0;
      if (chan_major) {
        const int row = row0 + lane;
        cm_ok = row < p.m;
        cm_row_in = cm_ok;
        if (conv) {
          const int per = p.conv_hp * p.conv_wp;
          const int smp = row / per, rem = row - smp * per;
          cm_smp = smp;
          const int yq = rem / p.conv_wp;
          const int yy = yq - p.conv_pad, xx = rem - yq * p.conv_wp - p.conv_pad;
          cm_ok = cm_ok && yy >= 0 && yy < p.conv_h && xx >= 0 && xx < p.conv_w;
          cm_stride = static_cast<long long>(p.conv_h) * p.conv_w;
          cm_o0 = static_cast<long long>(smp) * p.n * cm_stride + static_cast<long long>(yy) * p.conv_w + xx;
        } else {
          const long long smp = row / p.ohw;
          cm_smp = static_cast<int>(smp);
          cm_stride = p.ohw;
          cm_o0 = smp * p.n * cm_stride + (row - smp * p.ohw);
        }
      }
      // one 32-column chunk of this lane's row: scale, bias, activation, residual, stores
      auto process = [&](const int c0, const int col0, float (&v)[32]) {
        (void)c0;
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= p.acc_scale;
        const bool full_cols = (col0 + 32 <= p.n);
        // bias: the same 32 values for every lane (broadcast loads)
        if (p.bias != nullptr) {
          if (full_cols && ((reinterpret_cast<uintptr_t>(p.bias + col0) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 b4 = __ldg(reinterpret_cast<const float4*>(p.bias + col0 + j));
              v[j] += b4.x; v[j + 1] += b4.y; v[j + 2] += b4.z; v[j + 3] += b4.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.n) v[j] += __ldg(p.bias + col0 + j);
          }
        }
        switch (p.activation) {  // hoisted out of the element loop
          case MIMIR_B200_ELT_GELU:
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_ref(v[j]);
            break;
          case -1:
            break;
          default:
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.activation);
            break;
        }
        if (chan_major) {
          if (cm_ok) {
            const long long o0 = cm_o0 + static_cast<long long>(col0) * cm_stride;
            if (p.residual != nullptr) {
              // all loads first: the output may alias nothing here, but the compiler cannot know, and
              // load -> store -> load chains would serialise on memory latency
              float q[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) q[j] = (full_cols || col0 + j < p.n) ? __ldg(p.residual + o0 + j * cm_stride) : 0.0f;
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += q[j];
            }
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full_cols || col0 + j < p.n) p.out_f32[o0 + j * cm_stride] = v[j];
          }
          if (CM == 2 && p.gn_part != nullptr && row0 < p.m && col0 < p.n) {  // warp-uniform
            float* gd = p.gn_part + (static_cast<long long>(row0 >> 5) * ((p.n + 31) >> 5) + (col0 >> 5)) * (2 * (1 + 64 / p.gn_cpg));
            gn_emit_chunk(v, cm_ok, cm_row_in, cm_smp, min(32, p.n - col0), lane, p.gn_cpg, gd);
          }
        } else {
          // row-major: this lane owns 32 consecutive columns of its row = one 128-byte line, moved with
          // 256-bit loads / stores (full 32-byte sectors, no transposition needed)
          const int row = row0 + lane;
          if (row < p.m) {
            const long long ro = static_cast<long long>(row) * p.ldo + col0;
            if (p.residual != nullptr) {
              const float* rr = p.residual + ro;
              if (full_cols && ((reinterpret_cast<uintptr_t>(rr) & 31) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  float q[8];
                  ld_global_v8(rr + j, q);
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[j + e] += q[e];
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.n) v[j] += __ldg(rr + j);
              }
            }
            if (p.out_f32 != nullptr && !p.tma_store) {
              float* o = p.out_f32 + ro;
              if (full_cols && ((reinterpret_cast<uintptr_t>(o) & 31) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) st_global_v8(o + j, &v[j]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.n) o[j] = v[j];
              }
            }
            if (p.out_split != nullptr) {
              // hi/lo planes for the next GEMM; columns n..np-1 are written as zero so that the padded
              // K of the consumer stays zero (np is a multiple of 64, so the chunk is always whole)
              uint32_t hi[16], lo[16];
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                const float x0 = (full_cols || col0 + j < p.n) ? v[j] : 0.0f;
                const float x1 = (full_cols || col0 + j + 1 < p.n) ? v[j + 1] : 0.0f;
                split_pair(x0, x1, p.f16, hi[j >> 1], lo[j >> 1]);
              }
              __nv_bfloat16* oh = p.out_split + static_cast<long long>(row) * p.np + col0;
              __nv_bfloat16* ol = oh + static_cast<long long>(p.m) * p.np;
              st_global_v8_b32(oh, &hi[0]);
              st_global_v8_b32(oh + 16, &hi[8]);
              st_global_v8_b32(ol, &lo[0]);
              st_global_v8_b32(ol + 16, &lo[8]);
            }
          }
          if (p.tma_store) {
            // fp32 rows through a TMA store: staged in shared memory (128-byte swizzle, conflict-free 128-bit writes)
            // the 32 x 32 chunk is one copy, clipped at the edges of the output by the tensor map.
            float* tile = reinterpret_cast<float*>(epi_tiles + ew * 4096);
            if (lane == 0) bulk_wait_read0();  // the previous chunk's copy has read the tile
            __syncwarp();
#pragma unroll
            for (int c = 0; c < 8; ++c)
              *reinterpret_cast<float4*>(tile + lane * 32 + ((c ^ (lane & 7)) << 2)) = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&map_o, tile, col0, row0);
              bulk_commit();
            }
          }
        }
      };
      // (Tried: the next chunk's tensor-memory load in flight while this one is processed - two register sets, the
      // plain form has the room.  Measured neutral to 7 % slower on the K = 768 layers: the load's latency is not what
      // the short-K tiles wait for; operand and store bytes per MMA cycle are.)
      const int nch = (p.bn / 32) / 2;
#pragma unroll 1
      for (int ci = 0; ci < nch; ++ci) {
        const int c0 = (half * (p.bn / 64) + ci) * 32;
        const int col0 = tn * p.bn + c0;
        if (col0 >= col_limit) break;  // warp-uniform
        float v[32];
        tmem_ld_32x32(taddr0 + c0, v);
        process(c0, col0, v);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty[acc]), 0));  // the leader's MMA thread waits for both CTAs
        else mbar_arrive(&acc_empty[acc]);
      }
      if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1; }
    }
    if (lane == 0) bulk_wait_read0();  // no copy may still be reading shared memory when the CTA exits
  }

  tcgen05_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still signal it
  if (warp == 1) {
    tcgen05_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------
// fp32 -> bf16 hi/lo planes
// ------------------------------------------------------------------------------------------
namespace {

// One thread per 8 consecutive K elements of one row; the padded tail kp > k is written as zero.
__global__ void split_rows_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long rows, int k,
                                  int kp, int planes, int f16, float scale) {
  const int chunks = kp >> 3;
  const long long total = rows * chunks;
  const long long plane_stride = rows * static_cast<long long>(kp);
  const bool vec_ok = ((k & 3) == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / chunks;
    const int c = static_cast<int>(i - r * chunks) << 3;
    float v[8];
    const float* s = src + r * k + c;
    if (vec_ok && c + 8 <= k) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(s));
      const float4 b = __ldg(reinterpret_cast<const float4*>(s + 4));
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (c + j < k) ? __ldg(s + j) : 0.0f;
    }
    uint32_t h[4], l[4];
#pragma unroll
    for (int j = 0; j < 8; j += 2) split_pair(v[j] * scale, v[j + 1] * scale, f16, h[j >> 1], l[j >> 1]);
    __nv_bfloat16* d = dst + r * kp + c;
    *reinterpret_cast<uint4*>(d) = make_uint4(h[0], h[1], h[2], h[3]);
    if (planes == 2) *reinterpret_cast<uint4*>(d + plane_stride) = make_uint4(l[0], l[1], l[2], l[3]);
  }
}

// src fp32 [k, n] row-major -> planes of the transpose [n, kp].  32x32 tiles through shared memory.
__global__ void split_transposed_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int k, int n,
                                        int kp, int planes, int f16, float scale) {
  __shared__ float tile[32][33];
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int kk = k0 + i, nn = n0 + threadIdx.x;
    tile[i][threadIdx.x] = (kk < k && nn < n) ? __ldg(src + static_cast<long long>(kk) * n + nn) : 0.0f;
  }
  __syncthreads();
  const long long plane_stride = static_cast<long long>(n) * kp;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int nn = n0 + i, kk = k0 + threadIdx.x;
    if (nn < n && kk < kp) {
      uint16_t h, l;
      split_one(tile[threadIdx.x][i] * scale, f16, h, l);
      uint16_t* d16 = reinterpret_cast<uint16_t*>(dst);
      d16[static_cast<long long>(nn) * kp + kk] = h;
      if (planes == 2) d16[plane_stride + static_cast<long long>(nn) * kp + kk] = l;
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 3-D map over bf16 planes [planes][rows][kp]; box = {bk, box_rows, 1}; swizzle span = bk * 2 bytes.
int make_plane_map(CUtensorMap* map, const void* base, int planes, long long rows, int kp, int bk, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(MIMIR_B200_E_CUDA, "cuTensorMapEncodeTiled entry point not available");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail(MIMIR_B200_E_INVALID, "GEMM operand not 16-byte aligned");
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(kp), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(planes)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(kp) * 2, static_cast<cuuint64_t>(rows) * kp * 2};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(bk), static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapSwizzle sw = (bk == 64) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MIMIR_B200_E_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
  return MIMIR_B200_OK;
}

// 2-D map over the fp32 row-major output [rows][ld]; box = 32 x 32, 128-byte swizzle (the epilogue's staging tile)
int make_out_map(CUtensorMap* map, const float* base, long long rows, int cols, long long ld) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(MIMIR_B200_E_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MIMIR_B200_E_CUDA, "cuTensorMapEncodeTiled (output) failed (%d)", static_cast<int>(r));
  return MIMIR_B200_OK;
}

int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}

template <int BK>
int launch_gemm_t(const GemmArgs& g, cudaStream_t st) {
  const int kp = round_up(g.k, 64);
  const bool conv = g.conv_ks > 0;
  CUtensorMap map_a, map_w;
  // conv: A rows are `conv_c` channels long and K = taps * conv_c runs over (tap, channel)
  // narrow channel-major layers run with the operands swapped (see GemmParams::swap); short K keeps the usual
  // form, whose epilogue writes NCHW with coalesced stores
  const char* noswap = getenv("MIMIR_B200_GEMM_NOSWAP");
  const int kblocks_all = conv ? g.conv_ks * g.conv_ks * (g.conv_c / BK) : kp / BK;
  const bool swap = (conv || g.out_nchw_hw > 0) && g.n <= BM && g.bias == nullptr && g.out_split == nullptr && g.out_f32 != nullptr &&
                    g.m >= 4 * BN && kblocks_all * BK >= 256 && !(noswap && noswap[0] == '1');
  MB_TRY(make_plane_map(&map_a, g.a, g.a_planes, g.m, conv ? g.conv_c : kp, BK, swap ? BN : BM));
  // Optional (MIMIR_B200_GEMM_TMA_STORE=1): row-major fp32 outputs leave through TMA stores.  Measured neutral on the
  // decoder's K = 768 layers (1 078 vs 1 100 TFLOP/s issued): what slows those layers is not the shape of the stores but
  // their bytes - the operand loads alone run at ~62 B per cycle and SM, next to what an SM can take from L2, and the
  // same kernel without any output store reaches 1 315.
  static const bool use_tma_store = [] { const char* e = getenv("MIMIR_B200_GEMM_TMA_STORE"); return e && e[0] == '1'; }();
  const bool tma_store = use_tma_store && !swap && !conv && g.out_nchw_hw <= 0 && g.out_f32 != nullptr && g.ldo % 4 == 0 &&
                         (reinterpret_cast<uintptr_t>(g.out_f32) & 15) == 0;
  CUtensorMap map_o = map_a;  // (a valid map when unused)
  if (tma_store) MB_TRY(make_out_map(&map_o, g.out_f32, g.m, g.n, g.ldo));
  GemmParams p;
  p.tma_store = tma_store ? 1 : 0;
  p.swap = swap ? 1 : 0;
  p.tiles_m = swap ? (g.n + BM - 1) / BM : (g.m + BM - 1) / BM;
  p.bn = BN;
  if (!swap && !conv && !tma_store) {
    // MIMIR_B200_GEMM_BN=192: 192-column tiles.  On paper they shorten launches whose last wave is mostly empty (N = 768
    // over 256 row tiles: 7 waves of 192 columns instead of 6 of 256, 12.5 % less work per SM); measured, the
    // 32768 x 768 x 768 projection takes 0.076 ms either way and the K = 3072 one 0.243 against 0.251: an N = 192
    // instruction costs the tensor pipe about what an N = 256 one does.  Kept as a switch, off by default.
    static const int force = env_int("MIMIR_B200_GEMM_BN", 0);
    if (force == 192) p.bn = 192;
  }
  // CTA pairs: every form but the swapped one, full-width tiles.  Taken by default where they were measured to pay: launches of at least one
  // full wave of tiles in the modes with two or three MMAs per product (same-run A/B: the K = N = 4096 layer 14.9-15.0
  // -> 14.5 ms per three-layer step = 0.333 of the sustained peak, the whole ceiling of the three-MMA scheme; the decoder
  // step 18.51 -> 18.2 ms).  The one-MMA mode (14.78 -> 14.88 ms) and launches of a few tiles (the registry
  // transformer's 1024-row layers: 0.290 -> 0.295 ms per step) are better off alone.  MIMIR_B200_GEMM_PAIR=0 turns pairs
  // off, =1 takes them wherever the form allows.
  static const int pair_env = env_int("MIMIR_B200_GEMM_PAIR", -1);
  const bool pair_can = !swap && !tma_store && p.bn == BN && p.tiles_m >= 2 && g.a_group_rows <= 0;
  const long long tiles_all = static_cast<long long>(p.tiles_m) * ((g.n + BN - 1) / BN);
  const bool pair = pair_can && (pair_env == 1 || (pair_env != 0 && g.a_planes + g.w_planes >= 3 && tiles_all >= ctx().sm_count));
  if (g.a_group_rows > 0 && (swap || conv || g.out_nchw_hw > 0 || g.a_group_rows % BM != 0 || g.w_group_rows <= 0 ||
                             g.w_rows_total < static_cast<long long>((g.m + g.a_group_rows - 1) / g.a_group_rows - 1) * g.w_group_rows + g.n))
    return fail(MIMIR_B200_E_INVALID, "gemm: bad grouped-form arguments");
  MB_TRY(make_plane_map(&map_w, g.w, g.w_planes, g.a_group_rows > 0 ? g.w_rows_total : g.n, kp, BK, swap ? BM : (pair ? BN / 2 : p.bn)));
  p.m = g.m;
  p.n = g.n;
  p.kblocks = conv ? g.conv_ks * g.conv_ks * (g.conv_c / BK) : kp / BK;
  p.conv_ks = g.conv_ks;
  p.conv_cblocks = conv ? g.conv_c / BK : 1;
  p.conv_pad = g.conv_pad;
  p.conv_hp = g.conv_h + 2 * g.conv_pad;
  p.conv_wp = g.conv_w + 2 * g.conv_pad;
  p.conv_h = g.conv_h;
  p.conv_w = g.conv_w;
  p.a_planes = g.a_planes;
  p.w_planes = g.w_planes;
  p.tiles_n = swap ? (g.m + BN - 1) / BN : (g.n + p.bn - 1) / p.bn;
  if (pair) p.tiles_m = (p.tiles_m + 1) / 2;  // row PAIRS: the CTA of rank r takes row tile 2 * pair + r
  p.group_n = env_int("MIMIR_B200_GEMM_GROUP_N", 8);
  if (p.group_n < 1) p.group_n = 1;
  if (p.group_n > p.tiles_n) p.group_n = p.tiles_n;
  p.bias = g.bias;
  p.residual = g.residual;
  p.activation = g.activation;
  p.out_f32 = g.out_f32;
  p.ldo = g.ldo;
  p.out_split = g.out_split;
  p.np = round_up(g.n, 64);
  p.ohw = g.out_nchw_hw;
  p.err_word = ctx().dev_error_word;
  p.gn_part = nullptr;
  p.gn_cpg = 0;
  if (g.gn_part != nullptr) {
    if (!(g.conv_ks > 0 || g.out_nchw_hw > 0) || !(g.gn_cpg == 4 || g.gn_cpg == 8 || g.gn_cpg == 16 || g.gn_cpg == 32))
      return fail(MIMIR_B200_E_INVALID, "GEMM: GroupNorm partials need a channel-major output and 4, 8, 16 or 32 channels per group");
    p.gn_part = g.gn_part;
    p.gn_cpg = g.gn_cpg;
  }
  p.a_group_rows = g.a_group_rows;
  p.w_group_rows = g.w_group_rows;
  {
    // Measured on B200 against fp64 products of the same operand planes (random normal operands, K = 256 ... 4096,
    // two and three MMAs per 16-wide K step): the accumulated result is low by 1.47e-8 ... 1.58e-8 of its value per
    // MMA instruction that added into it; all-positive operands lose 2.1e-8 ... 3.6e-8.  Zero-padded K adds exact
    // zeros and loses nothing, so only the real K counts.  Undoing the mean loss halves the accumulation error.
    const long long ksteps = conv ? static_cast<long long>(g.conv_ks) * g.conv_ks * ((g.conv_c + UMMA_K - 1) / UMMA_K)
                                  : (g.k + UMMA_K - 1) / UMMA_K;
    const int products = 1 + (g.a_planes == 2 ? 1 : 0) + (g.w_planes == 2 ? 1 : 0);
    static const bool comp = [] { const char* e = getenv("MIMIR_B200_ACC_COMP"); return !(e && e[0] == '0'); }();
    p.acc_scale = (comp ? 1.0f + ACC_TRUNC_PER_MMA * static_cast<float>(ksteps * products) : 1.0f) / g.w_scale;
  }
  p.f16 = plane_format() == PLANES_F16 ? 1 : 0;
  constexpr int RING_BYTES = 196608;  // 192 KB of operand stages, cut into as many stages as the planes in use allow
  constexpr int SMEM = RING_BYTES + 1024 /*align slack*/ + 512 /*barriers*/ + EPI_WARPS * 32 * 33 * 4 /*swapped-epilogue tiles*/;
  static_assert(SMEM <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
  {
    const int m_pl = swap ? g.w_planes : g.a_planes, n_pl = swap ? g.a_planes : g.w_planes;
    p.stage_bytes = m_pl * BM * BK * 2 + n_pl * (pair ? BN / 2 : BN) * BK * 2;
    p.stages = RING_BYTES / p.stage_bytes;
    if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
    const int want = env_int("MIMIR_B200_GEMM_STAGES", 0);
    if (want >= 2 && want < p.stages) p.stages = want;
  }
  const bool cm = swap || conv || g.out_nchw_hw > 0;
  // CM = 2: the channel-major form with the GroupNorm partials compiled into its epilogue (a form of its own, so that the
  // convolutions that do not emit them run the code they always ran)
  auto kern = cm ? (p.gn_part != nullptr
                        ? (pair ? gemm_tn_bf16split_kernel<BK, RING_BYTES, 2, 1> : gemm_tn_bf16split_kernel<BK, RING_BYTES, 2, 0>)
                        : (pair ? gemm_tn_bf16split_kernel<BK, RING_BYTES, 1, 1> : gemm_tn_bf16split_kernel<BK, RING_BYTES, 1, 0>))
                 : (pair ? gemm_tn_bf16split_kernel<BK, RING_BYTES, 0, 1> : gemm_tn_bf16split_kernel<BK, RING_BYTES, 0, 0>);
  static PerDeviceOnce attr_once;
  MB_TRY(attr_once.run([&]() -> int {
    MB_CUDA(cudaFuncSetAttribute(gemm_tn_bf16split_kernel<BK, RING_BYTES, 0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    MB_CUDA(cudaFuncSetAttribute(gemm_tn_bf16split_kernel<BK, RING_BYTES, 1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    MB_CUDA(cudaFuncSetAttribute(gemm_tn_bf16split_kernel<BK, RING_BYTES, 0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    MB_CUDA(cudaFuncSetAttribute(gemm_tn_bf16split_kernel<BK, RING_BYTES, 1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    MB_CUDA(cudaFuncSetAttribute(gemm_tn_bf16split_kernel<BK, RING_BYTES, 2, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    MB_CUDA(cudaFuncSetAttribute(gemm_tn_bf16split_kernel<BK, RING_BYTES, 2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    return MIMIR_B200_OK;
  }));
  const int tiles = p.tiles_m * p.tiles_n;
  int grid = tiles < ctx().sm_count ? tiles : ctx().sm_count;
  if (pair) {
    const int pairs = ctx().sm_count / 2;
    grid = 2 * (tiles < pairs ? tiles : pairs);
  }
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (ctx().prof_gemm) {
    MB_CUDA(cudaEventCreate(&e0));
    MB_CUDA(cudaEventCreate(&e1));
    MB_CUDA(cudaEventRecord(e0, st));
  }
  if (pair) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MB_CUDA(cudaLaunchKernelEx(&cfg, kern, map_a, map_w, map_o, p));
  } else {
    kern<<<grid, NUM_THREADS, SMEM, st>>>(map_a, map_w, map_o, p);
  }
  MB_CUDA(cudaGetLastError());
  if (e0) {
    MB_CUDA(cudaEventRecord(e1, st));
    ctx().prof_events.push_back(e0);
    ctx().prof_events.push_back(e1);
  }
  count_launch();
  return MIMIR_B200_OK;
}

}  // namespace

int plane_format() {
  static const int fmt = [] {
    const char* e = getenv("MIMIR_B200_PLANES");
    return (e && (e[0] == 'b' || e[0] == 'B')) ? PLANES_BF16 : PLANES_F16;
  }();
  return fmt;
}

namespace {
// largest finite |w| as its bit pattern (non-negative floats order like unsigned integers)
__global__ void absmax_kernel(const float* __restrict__ w, size_t n, unsigned* __restrict__ out) {
  unsigned m = 0;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const unsigned u = __float_as_uint(__ldg(w + i)) & 0x7fffffffu;
    if (u < 0x7f800000u && u > m) m = u;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, d));
  if ((threadIdx.x & 31) == 0 && m != 0) atomicMax(out, m);
}
}  // namespace

int weight_plane_scale(const float* w_dev, size_t n, cudaStream_t st, float* scale) {
  *scale = 1.0f;
  if (plane_format() != PLANES_F16 || n == 0 || w_dev == nullptr) return MIMIR_B200_OK;
  static std::mutex mu;  // one spare device word is shared by every caller
  std::lock_guard<std::mutex> lk(mu);
  unsigned* word = reinterpret_cast<unsigned*>(ctx().dev_error_word) + 8;  // a spare word of the 256-byte error block
  MB_CUDA(cudaMemsetAsync(word, 0, sizeof(unsigned), st));
  const size_t want = (n + 255) / 256;
  const int blocks = static_cast<int>(want < static_cast<size_t>(ctx().sm_count) * 8 ? want : static_cast<size_t>(ctx().sm_count) * 8);
  absmax_kernel<<<blocks, 256, 0, st>>>(w_dev, n, word);
  MB_CUDA(cudaGetLastError());
  count_launch();
  unsigned bits = 0;
  MB_CUDA(cudaMemcpyAsync(&bits, word, sizeof(unsigned), cudaMemcpyDeviceToHost, st));
  MB_CUDA(cudaStreamSynchronize(st));
  float amax;
  memcpy(&amax, &bits, sizeof(float));
  if (!(amax > 0.0f)) return MIMIR_B200_OK;
  int e = 0;
  frexpf(amax, &e);            // amax = f * 2^e with f in [0.5, 1)
  int s = 14 - e;              // amax * 2^s in [2^13, 2^14)
  if (s > 60) s = 60;
  if (s < -60) s = -60;
  *scale = ldexpf(1.0f, s);
  return MIMIR_B200_OK;
}

int launch_split(const float* src, __nv_bfloat16* dst, int64_t rows, int k, int planes, cudaStream_t st, float scale) {
  if (rows <= 0 || k <= 0) return MIMIR_B200_OK;
  const int kp = round_up(k, 64);
  const long long total = rows * (kp >> 3);
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  const long long cap = static_cast<long long>(ctx().sm_count) * 16;
  if (blocks > cap) blocks = cap;
  split_rows_kernel<<<static_cast<int>(blocks), threads, 0, st>>>(src, dst, rows, k, kp, planes, plane_format() == PLANES_F16, scale);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_split_transposed(const float* src, __nv_bfloat16* dst, int k, int n, int planes, cudaStream_t st, float scale) {
  if (n <= 0 || k <= 0) return MIMIR_B200_OK;
  const int kp = round_up(k, 64);
  dim3 grid((n + 31) / 32, kp / 32), block(32, 8);
  split_transposed_kernel<<<grid, block, 0, st>>>(src, dst, k, n, kp, planes, plane_format() == PLANES_F16, scale);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

namespace {
// One CTA that waits on an mbarrier nobody arrives on, with the kernels' own bounded wait and a caller-given limit:
// the wait runs out, the error word and the abort flag are set, the roles leave, the TMEM columns are freed and the
// kernel returns - the give-up path of the tensor-core kernels, run on purpose.
__global__ void __launch_bounds__(64) wait_timeout_selftest_kernel(unsigned long long limit_ns, int* err_word) {
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, 32);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (warp == 0) {
    // the same whole-warp form the epilogue and softmax warps use: lane 0 waits, the verdict is made warp-uniform
    int ok = 1;
    if (lane == 0) ok = mbar_wait_limit(&bar, 0, &abort_flag, err_word, 90, limit_ns, 0xF) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    (void)ok;
  } else if (lane == 0) {
    // a second role that sees the first one's abort flag and leaves (or runs out itself)
    mbar_wait_limit(&bar, 0, &abort_flag, err_word, 91, 4 * limit_ns, 0xF);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
}
}  // namespace

int launch_wait_timeout_selftest(unsigned long long limit_ns, cudaStream_t st) {
  if (limit_ns == 0 || limit_ns > 100000000ull) return fail(MIMIR_B200_E_INVALID, "selftest: the limit must be within (0, 100 ms]");
  wait_timeout_selftest_kernel<<<1, 64, 0, st>>>(limit_ns, ctx().dev_error_word);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_gemm(const GemmArgs& g, cudaStream_t st) {
  if (g.m <= 0 || g.n <= 0 || g.k <= 0) return fail(MIMIR_B200_E_INVALID, "gemm: empty dimension");
  if (!g.a || !g.w) return fail(MIMIR_B200_E_INVALID, "gemm: null operand");
  if (!g.out_f32 && !g.out_split) return fail(MIMIR_B200_E_INVALID, "gemm: no output");
  if (g.residual && !g.out_f32) return fail(MIMIR_B200_E_INVALID, "gemm: residual needs the fp32 output stride");
  // K block per stage.  With at most three planes in play (one of the operands single-plane) a 64-wide block still leaves
  // three 64 KB stages, halves the barrier round trips per MMA and uses 128-byte swizzle rows: measured on the decoder's
  // K = 768 layers 0.77 -> 0.90 of the sustained cuBLAS rate.  With four planes (both operands split) 64-wide blocks would
  // leave two 96 KB stages, which measured slower than four 48 KB stages of 32.
  if (g.conv_ks > 0) {
    if (g.conv_c <= 0 || g.conv_c % 32 != 0 || g.k != g.conv_ks * g.conv_ks * g.conv_c || g.out_split || !g.out_f32)
      return fail(MIMIR_B200_E_INVALID, "gemm: bad shifted-convolution arguments");
  }
  const int bk = env_int("MIMIR_B200_GEMM_BK", (g.a_planes + g.w_planes <= 3) ? 64 : 32);
  if (bk == 64 && (g.conv_ks == 0 || g.conv_c % 64 == 0)) return launch_gemm_t<64>(g, st);
  return launch_gemm_t<32>(g, st);
}

}  // namespace mb
