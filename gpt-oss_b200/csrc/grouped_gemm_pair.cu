// Grouped expert GEMMs on CTA pairs (tcgen05 cta_group::2), weights as the M
// operand.
//
// Same math and same outputs as grouped_gemm.cu, computed transposed:
//   D^T[n, j] = sum_k W[e][n, k] * X[tok0 + j, k]
// A pair of CTAs (one cluster of 2, the two SMs of a TPC) owns 256 weight rows of
// one expert (128 per CTA, the MMA's M) and a tile of up to 256 of that expert's
// tokens (the MMA's N, any multiple of 16).  Each CTA loads its own 128 weight
// rows and its own half of the token tile - 32 KB per 64-deep K block instead of
// the 46 KB of the single-CTA kernel - and the even CTA issues one
// tcgen05.mma.cta_group::2 (M=256, N=tokens) that reads both CTAs' shared memory
// and writes 128 accumulator rows into each CTA's TMEM.  What this buys:
//   * a third less L2->SM and shared-memory traffic per flop (the single-CTA
//     kernel is bound by it, not by the tensor pipe);
//   * no ragged-M waste: the last token tile of an expert is as narrow as the
//     expert's rows need (rounded up to 16), so 192 rows per expert (120b shape)
//     or a handful (decode shapes) cost their own N, not a 128-row tile;
//   * each expert's weights are the streamed operand, read once per token tile.
// No TMA load uses multicast: the halves of the shared operand are loaded by the
// CTA that holds them.
//
// Warp roles per CTA (320 threads): warp 0 = TMA producer (both CTAs; the odd
// CTA's loads complete on the even CTA's full barrier), warp 1 of the even CTA =
// MMA issuer, warp 1 = paired TMEM allocation, warps 2-9 = epilogue.  The producer
// and the issuer walk their rings with the whole warp - every lane polls the
// barriers - and one lane picked by elect.sync inside the loop body issues.  (With
// `if (lane == 0)` around the whole loop each TMA, MMA and commit cost the lone lane
// 60-70 cycles to issue: a K block took 630-680 cycles whatever it contained, against
// 450-530 this way.)  tcgen05.commit with a 2-CTA mask releases the stage / publishes
// the accumulator in both CTAs; the odd CTA's epilogue warps release the accumulator
// with a remote mbarrier arrive.
//
// Epilogue (transposed): a TMEM lane is an output feature, a column a token.  A
// warp reads 32 lanes x 32 tokens, adds the lane's bias, pairs gate/up rows
// (adjacent lanes) by shuffle or applies the token's routing weight, and writes
// bf16 into a [32 tokens][row] shared tile shared by the 4 warps that cover the
// CTA's 128 rows; the tile then leaves row-wise, one bulk copy per token (a whole
// 128- / 256-byte segment), to this GPU's memory or - down GEMM under expert
// parallelism, GemmArgs::row_dst - straight into the memory of the rank the token
// came from.
#include <cuda.h>

#include "common.cuh"
#include "engine.h"
#include "gemm_epilogue.cuh"
#include "umma_2sm.cuh"

namespace gptoss {

constexpr int kPairThreads = 320;
constexpr int kPairOperandBytes = 128 * kTileK * 2;          // 16 KB: 128 rows x 64 k
constexpr int kPairEpiWarps = kPairThreads / 32 - 2;
constexpr int kAccColsPair = 256;  // TMEM columns per accumulator (up to 256 tokens), two of them

template <int EPI>
struct PairStage {
  // per token, per CTA: 64 activations, 128 bf16 outputs or 128 fp32 outputs
  static constexpr int kRowBytes = (EPI == kEpiSwiglu) ? 128 : (EPI == kEpiF32 ? 512 : 256);
  // 16 bytes of padding keep the 2-byte writes of the SwiGLU epilogue off each
  // other's banks; the 256-byte rows of the down epilogue go unpadded so that six
  // operand stages still fit
  static constexpr int kPitch = (EPI == kEpiSwiglu) ? kRowBytes + 16 : kRowBytes;
  static constexpr int kTileBytes = 32 * kPitch;
  static constexpr int kTotalBytes = 2 /*halves*/ * 2 /*buffers*/ * kTileBytes;
};

// MXFP4 weights (MX = true): a producer warp bulk-copies the packed codes (4 KB) and
// scales (256 B) of the CTA's 128 rows x 64 k into a raw ring; sixteen extra warps expand
// them to bf16 straight into the operand ring, in the 128-byte-swizzled layout TMA would
// have written, and count as arrivals on the even CTA's full barrier beside the token
// tiles' bytes.  The expansion is register arithmetic only (a table in shared memory cost
// more shared-memory cycles per K block than the MMAs' own operand reads): per code pair a
// mask, a multiply, a mask and the multiply by the block scale.
//
// Decode-sized batches (token tiles of at most 64 rows, template flag TA) go one step
// further.  With so few tokens a K block holds little work of any kind and the hand-shakes
// around it - four rings, each with a wait, an issue and an arrival or a commit per K
// block - are most of its time: with the expansion's arithmetic, the MMAs, the token loads
// and even the weight loads from HBM all switched off, a launch still took 0.72 of its
// full time.  So (1) a ring stage carries kTaKbs = 3 K blocks: one raw copy, one round of
// waits and one commit per 192 k; (2) the expanded weights go to tensor memory, not to
// shared memory: a lane expands one weight row and stores it into its own TMEM lane
// (tcgen05.st), and the MMA takes its M operand from there.  The accumulators need only
// 2 x 64 columns, which leaves 384 for four stages of 3 x 32 columns of weights; shared
// memory holds the raw ring and the token tiles only.
constexpr int kPairBarrierBytes = 1024;  // mbarriers, TMEM address holder, abort flag
constexpr int kRawCodeBytes = 128 * 32;
constexpr int kRawStageBytes = kRawCodeBytes + 128 * 2;
// Expanding warps: groups of four; group j takes the K blocks n = j, j + G, j + 2G, ... of
// the CTA's sequence (G groups).  With up to four operand stages there is a group per stage;
// with six, three groups alternate between two stages each (n % 6), so a group starts on its
// next block while the MMAs still read its last one - otherwise the stage's round trip
// (expand, MMAs, commit, wake-up) sets the pace, not the expansion.
constexpr int kDqGroupWarps = 4;
constexpr int kTaKbs = 3;  // K blocks per ring stage when the weights go to TMEM (TA)
__host__ __device__ constexpr int dq_groups(int stages) { return stages > 4 ? stages / 2 : stages; }
__host__ __device__ constexpr int dq_warps(int stages) { return dq_groups(stages) * kDqGroupWarps; }

// two e2m1 codes, one in bits 0-3 and one in bits 16-19 (kLow) or in bits 4-7 and 20-23
// (!kLow), all other bits zero -> two bf16 whose value is code * 2^-126: sign to bit 15 of
// its half, the three magnitude bits to exponent bits 0-1 and mantissa bit 6 (magnitude
// code 1 becomes the bf16 subnormal 2^-127, which bf16 multiplies take at full rate).  One
// multiply makes both shifted copies (by 6 and by 12, or by 2 and by 8; they cannot overlap),
// one mask keeps the bits that matter.
template <bool kLow>
__device__ __forceinline__ uint32_t e2m1_pair_to_bf16x2_raw(uint32_t u) {
  return (u * (kLow ? 0x1040u : 0x104u)) & 0x81C081C0u;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&a),
                             *reinterpret_cast<__nv_bfloat162 *>(&b));
  return *reinterpret_cast<uint32_t *>(&r);
}

// Linear tile index -> (token tile, weight-row pair): the pairs of one token tile are
// consecutive, so the clusters of one wave share one or two token tiles (L2 hits) and stream
// each weight block once.  (Spreading a wave over several token tiles measured no faster.)
__device__ __forceinline__ void decode_tile(int tile, int w_pairs, int tt_lo, int *tt, int *wp) {
  const int q = tile / w_pairs;
  *tt = tt_lo + q;
  *wp = tile - q * w_pairs;
}

// TOKB = token rows a CTA's operand slot holds (128: token tiles of up to 256; 32:
// tiles of up to 64 for decode-sized batches, which buys a deeper ring)
// kRawStages = depth of the raw (packed) weight ring, 0 without MX
// TA = the expanded weights go to tensor memory, not to the operand ring (MX, decode-sized
// token tiles): see the dequantising warps below
template <int EPI, int kPairStages, bool MX, int TOKB, int kRawStages, bool TA>
__global__ void __launch_bounds__(kPairThreads + (MX ? (dq_warps(kPairStages) + 1) * 32 : 0), 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_w,
                         const __grid_constant__ CUtensorMap tmap_x,
                         const __grid_constant__ CUtensorMap tmap_x32,
                         const __grid_constant__ CUtensorMap tmap_x8, const GemmArgs g) {
  // K blocks per ring stage, i.e. per round of barrier hand-shakes.  With TA the hand-shakes
  // themselves (wait, issue, commit, wake-up on four rings) are most of a K block's time at
  // decode sizes, so a stage carries two K blocks: one raw copy, one wait and one commit per
  // 128 k (the last stage of an odd count carries one)
  constexpr int kKbs = TA ? kTaKbs : 1;
  constexpr int kTokOff = TA ? 0 : kPairOperandBytes;  // token half within a stage
  constexpr int kTokBytes = TOKB * kTileK * 2;          // one K block of the CTA's token half
  constexpr int kPairStageBytes = kTokOff + kKbs * kTokBytes;  // weights (unless TA) + tokens
  constexpr int kRawSlotBytes = kKbs * kRawStageBytes;
  // TMEM columns: two accumulators of up to 256 token columns; with TA the token tiles have
  // at most 64 rows, the accumulators sit 64 columns apart and the weight operand takes 32
  // columns (64 k as bf16 pairs) per K block from column 128 on
  constexpr int kAccStride = TA ? 64 : kAccColsPair;
  constexpr int kTmemACol0 = 128;
  constexpr int kTmemAStageCols = kKbs * 32;
  static_assert(!TA || (MX && TOKB == 32 && kTmemACol0 + kPairStages * kTmemAStageCols <= 512),
                "the TMEM-resident weight operand needs MX, 64-row token tiles and room in TMEM");
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + kPairStages * kPairStageBytes);
  uint64_t *empty_bar = full_bar + kPairStages;
  uint64_t *tfull_bar = empty_bar + kPairStages;  // [2]
  uint64_t *tempty_bar = tfull_bar + 2;           // [2], used in the even CTA
  uint64_t *raw_full = tempty_bar + 2;            // [kRawStages] (MX)
  uint64_t *raw_empty = raw_full + kRawStages;    // [kRawStages] (MX)
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(raw_empty + kRawStages);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);
  static_assert((2 * kPairStages + 4 + 2 * kRawStages) * 8 + 8 <= kPairBarrierBytes,
                "barrier region too small");
  unsigned char *epi_stage = smem + kPairStages * kPairStageBytes + kPairBarrierBytes;
  unsigned char *raw_ring = epi_stage + PairStage<EPI>::kTotalBytes;  // (MX)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  // (MX) operand stage s is always filled by the same kWarpsPerBlock dequantising warps,
  // and a raw stage always drained by the same ones: every warp then meets the phases of
  // its barriers one by one, in order, and a parity wait can never be a whole turn of
  // the ring ahead of the barrier it polls
  constexpr int kDequantWarps = dq_warps(kPairStages), kGroups = dq_groups(kPairStages);
  constexpr int kWarpsPerBlock = MX ? kDqGroupWarps : 1;
  static_assert(!MX || (kRawStages % kPairStages == 0 && kPairStages % kGroups == 0 &&
                        8 % kWarpsPerBlock == 0),
                "dequantising warps must map to fixed ring stages");

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; s++) {
      // MX: the leader's producer plus the dequantising warps of the block in each CTA
      mbar_init(&full_bar[s], MX ? 1 + 2 * kWarpsPerBlock : 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < kRawStages; s++) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], kWarpsPerBlock);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 2 * kPairEpiWarps);  // epilogue warps of both CTAs
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_barrier_all();  // the peer's barriers exist before anything targets them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // everything above touched no global memory: under a programmatic dependent launch it
  // ran while the previous kernel of the stream was still finishing
  grid_dependency_wait();
  grid_launch_dependents();

  const int w_pairs = (g.n_cols + 255) / 256;
  // token tiles of this launch: all of them, or one side of g.tile_split (the schedule is
  // ordered by expert, so a side is a range of experts)
  int tt_lo = 0, tt_hi = *g.num_mtiles;
  if (g.tile_part == 1) tt_hi = *g.tile_split;
  if (g.tile_part == 2) tt_lo = *g.tile_split;
  const int n_tt = tt_hi - tt_lo;
  const int first_tile = blockIdx.x >> 1;
  const int total_tiles = n_tt * w_pairs;
  const int kb_count = (g.k_dim + kTileK - 1) / kTileK;
  const int sb_count = (kb_count + kKbs - 1) / kKbs;  // ring stages per tile
  const int ncl = gridDim.x >> 1;  // clusters of the launch; a cluster strides over the tiles

  if (warp == 0) {
    {  // the whole warp walks the ring; one elected lane issues the loads
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int e_next = 0, tok0_next = 0, ntok_next = 0;
      bool sib_next = false;  // the expert has a second token tile, which re-reads its weights
      int tt, wp, tt2, wp2;
      auto has_sibling = [&](int t, int e) {
        return (t + 1 < tt_hi && g.mtile_expert[t + 1] == e) || (t > tt_lo && g.mtile_expert[t - 1] == e);
      };
      // an expert's weights pass through L2 once when all its rows fit one token tile: first
      // out (otherwise the expert's other token tiles, a few tiles further on in the same wave,
      // read them again: no hint); token tiles are re-read by every weight-row pair of the
      // expert: last out
      const uint64_t pol_once = g.l2_hints ? l2_policy_evict_first() : l2_policy_normal();
      const uint64_t pol_again = l2_policy_normal();
      const uint64_t pol_x = g.l2_hints ? l2_policy_evict_last() : l2_policy_normal();
      if (first_tile < total_tiles) {
        decode_tile(first_tile, w_pairs, tt_lo, &tt, &wp);
        e_next = g.mtile_expert[tt];
        tok0_next = g.mtile_row0[tt];
        ntok_next = g.mtile_rows[tt];
        sib_next = has_sibling(tt, e_next);
      }
      for (int tile = first_tile; ok && tile < total_tiles; tile += ncl) {
        decode_tile(tile, w_pairs, tt_lo, &tt, &wp);
        const int e = e_next, tok0 = tok0_next, ntok = ntok_next;
        const uint64_t pol_w = sib_next ? pol_again : pol_once;
        const int tile2 = tile + ncl;
        if (tile2 < total_tiles) {
          decode_tile(tile2, w_pairs, tt_lo, &tt2, &wp2);
          e_next = g.mtile_expert[tt2];
          tok0_next = g.mtile_row0[tt2];
          ntok_next = g.mtile_rows[tt2];
          sib_next = has_sibling(tt2, e_next);
        }
        const int half_n = ((ntok + 15) & ~15) >> 1;  // token rows each CTA contributes
        const int wrow = e * g.n_cols + wp * 256 + static_cast<int>(rank) * 128;
        const int trow = tok0 + static_cast<int>(rank) * half_n;
        // narrow token tiles are loaded with a narrower box: 8, 32 or 128 rows per CTA
        const CUtensorMap *tx =
            half_n <= 8 ? &tmap_x8 : ((half_n <= 32 || TOKB == 32) ? &tmap_x32 : &tmap_x);
        const uint32_t tok_bytes =
            (half_n <= 8 ? 8 : ((half_n <= 32 || TOKB == 32) ? 32 : 128)) * kTileK * 2;
        for (int sb = 0; sb < sb_count; sb++) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            set_status(g.status, kStatusWaitTimeoutProducer);
            *abort_flag = 1;
            ok = false;
            break;
          }
          unsigned char *sa = smem + stage * kPairStageBytes;
          const int kb = sb * kKbs;
          const int nkb = kb_count - kb < kKbs ? kb_count - kb : kKbs;
          if (elect_one()) {
            if (!MX) {
              if (rank == 0)
                mbar_arrive_expect_tx(&full_bar[stage], 2 * (kPairOperandBytes + tok_bytes));
              tma_load_2d_pair_hint(sa, &tmap_w, &full_bar[stage], kb * kTileK, wrow, pol_w);
            } else if (rank == 0) {
              // the weights arrive through the raw ring and the dequantising warps
              mbar_arrive_expect_tx(&full_bar[stage], 2 * tok_bytes * nkb);
            }
            for (int j = 0; j < nkb; j++)
              tma_load_2d_pair_hint(sa + kTokOff + j * kTokBytes, tx, &full_bar[stage],
                                    (kb + j) * kTileK, trow, pol_x);
          }
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (MX && warp == kPairThreads / 32 + kDequantWarps) {
    // raw-weight producer: one bulk copy (packed codes + scales of 128 rows x 64 k) per
    // K block into a ring deep enough to cover HBM latency at HBM bandwidth
    {
      int rs = 0;
      uint32_t rphase = 0;
      bool ok = true;
      for (int tile = first_tile; ok && tile < total_tiles; tile += ncl) {
        int tt, wp;
        decode_tile(tile, w_pairs, tt_lo, &tt, &wp);
        const int e = g.mtile_expert[tt];
        const size_t blk0 =
            (static_cast<size_t>(e) * (2 * w_pairs) + 2 * wp + rank) * kb_count;
        for (int sb = 0; sb < sb_count; sb++) {
          if (!mbar_wait(&raw_empty[rs], rphase ^ 1u, abort_flag)) {
            set_status(g.status, kStatusWaitTimeoutProducer);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const int kb = sb * kKbs;
          const int nkb = kb_count - kb < kKbs ? kb_count - kb : kKbs;
          if (elect_one()) {  // the K blocks of a tile follow each other in memory
            mbar_arrive_expect_tx(&raw_full[rs], nkb * kRawStageBytes);
            bulk_load(raw_ring + rs * kRawSlotBytes, g.wq + (blk0 + kb) * kRawStageBytes,
                      nkb * kRawStageBytes, &raw_full[rs]);
          }
          if (++rs == kRawStages) {
            rs = 0;
            rphase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // the whole warp walks the ring (every lane polls the barriers); one elected lane issues
    if (rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = first_tile; ok && tile < total_tiles; tile += ncl) {
        int tt, wp;
        decode_tile(tile, w_pairs, tt_lo, &tt, &wp);
        const int ntok = g.mtile_rows[tt];
        const uint32_t idesc = umma_idesc_bf16(256, (ntok + 15) & ~15);
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) {
          set_status(g.status, kStatusWaitTimeoutMma);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccStride;
        for (int sb = 0; sb < sb_count; sb++) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            set_status(g.status, kStatusWaitTimeoutMma);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kPairStageBytes);
          const uint64_t da = umma_smem_desc_sw128(sa);
          const int nkb = kb_count - sb * kKbs < kKbs ? kb_count - sb * kKbs : kKbs;
          if (elect_one()) {
            for (int j = 0; j < nkb; j++) {
              const uint64_t db = umma_smem_desc_sw128(sa + kTokOff + j * kTokBytes);
              const uint32_t ta = tmem_base + kTmemACol0 + stage * kTmemAStageCols + j * 32;
#pragma unroll
              for (int k = 0; k < kTileK / 16; k++) {
                if (TA)  // 16 k = 8 columns of the K block's 32
                  umma_bf16_pair_ta(d_tmem, ta + k * 8, db + 2 * k, idesc,
                                    (sb | j | k) != 0 ? 1u : 0u);
                else
                  umma_bf16_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (sb | k) != 0 ? 1u : 0u);
              }
            }
            umma_commit_pair(&empty_bar[stage], 3);  // frees the stage in both CTAs
          }
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (elect_one()) umma_commit_pair(&tfull_bar[acc], 3);  // accumulator ready in both CTAs
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (MX && warp >= kPairThreads / 32) {
    // dequantising warps: group j = dw / kWarpsPerBlock expands the K blocks n = j, j + G,
    // j + 2G, ... of the CTA's sequence into operand stage n % S, each warp of the group a
    // share of the block's 16-byte chunks.  Chunk c = half (c & 1) of weight row c >> 1:
    // 32 codes under one scale byte.
    const int dw = warp - kPairThreads / 32;
    const int grp = dw / kWarpsPerBlock, sub = dw - grp * kWarpsPerBlock;
    const int my_tiles = first_tile < total_tiles ? (total_tiles - first_tile + ncl - 1) / ncl : 0;
    const int total_kb = my_tiles * sb_count;  // ring stages this CTA passes through
    constexpr int kChunkIters = 8 / kWarpsPerBlock;
    if (grp < kGroups) {
      int sb = grp % sb_count;  // the stage's place within its tile
      for (int n = grp; n < total_kb; n += kGroups) {
        constexpr int kRawDiv = kRawStages > 0 ? kRawStages : 1;  // (no raw ring without MX)
        const int rs = n % kRawDiv;
        const uint32_t rphase = (n / kRawDiv) & 1;
        // a stage (and a raw slot) always meets the same group: n % S determines n % G
        const int stage = n % kPairStages;
        const uint32_t phase = (n / kPairStages) & 1;
        if (!mbar_wait(&raw_full[rs], rphase, abort_flag) ||
            !mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
          set_status(g.status, kStatusWaitTimeoutProducer);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();  // the MMAs that read this operand slot are done
        const unsigned char *rq = raw_ring + rs * kRawSlotBytes;
        unsigned char *slot = smem + stage * kPairStageBytes;
        const int nkb = kb_count - sb * kKbs < kKbs ? kb_count - sb * kKbs : kKbs;
        sb += kGroups;
        while (sb >= sb_count) sb -= sb_count;
        if (TA) {
          // A lane expands one whole weight row of the block (64 codes, two scales) and
          // stores it into its own TMEM lane: the warp's quarter of TMEM (warp index % 4)
          // decides which 32 rows it takes.  Column 16 h + 4 j + p of the stage holds
          // elements 32 h + 8 j + 2 p and + 1 of the row, the layout the MMA reads its M
          // operand in.  Nothing of the weights touches shared memory after the raw tile.
          const int qrow = (warp & 3) * 32 + lane;
          for (int jb = 0; jb < nkb; jb++) {
          const unsigned char *rqb = rq + jb * kRawStageBytes;
          const uint32_t sc2 =
              *reinterpret_cast<const unsigned short *>(rqb + kRawCodeBytes + 2 * qrow);
          const uint32_t taddr_a = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) +
                                   kTmemACol0 + stage * kTmemAStageCols + jb * 32;
#pragma unroll
          for (int hf = 0; hf < 2; hf++) {
            const uint4 q0 = *reinterpret_cast<const uint4 *>(rqb + (2 * qrow + hf) * 16);
            const uint32_t sc = (sc2 >> (8 * hf)) & 0xFFu;
            const uint32_t s1 = sc < 128u ? sc : 128u;
            const uint32_t m1 = (s1 + 126u) << 7;
            const uint32_t mul = m1 | (m1 << 16);
            const bool two = __any_sync(0xffffffffu, sc > 128u);
            const uint32_t m2 = (sc > 128u ? sc - 1u : 127u) << 7, mul2 = m2 | (m2 << 16);
            const uint32_t words[4] = {q0.x, q0.y, q0.z, q0.w};
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const uint32_t w = words[j], w8 = w >> 8;
              o[4 * j + 0] = bf16x2_mul(e2m1_pair_to_bf16x2_raw<true>(w & 0x000F000Fu), mul);
              o[4 * j + 1] = bf16x2_mul(e2m1_pair_to_bf16x2_raw<false>(w & 0x00F000F0u), mul);
              o[4 * j + 2] = bf16x2_mul(e2m1_pair_to_bf16x2_raw<true>(w8 & 0x000F000Fu), mul);
              o[4 * j + 3] = bf16x2_mul(e2m1_pair_to_bf16x2_raw<false>(w8 & 0x00F000F0u), mul);
            }
            if (two) {
#pragma unroll
              for (int j = 0; j < 16; j++) o[j] = bf16x2_mul(o[j], mul2);
            }
            tmem_st16(taddr_a + 16 * hf, o);
          }
          }
          tmem_st_wait();
          tc_fence_before();
        } else {
#pragma unroll
          for (int i = 0; i < kChunkIters; i++) {
            const int c = (sub * kChunkIters + i) * 32 + lane;
            const int wr = c >> 1, hf = c & 1;
            const uint4 q0 = *reinterpret_cast<const uint4 *>(rq + c * 16);
            const uint32_t sc = rq[kRawCodeBytes + c];
            // the bit trick leaves code * 2^-126; times 2^126 * 2^(s-127) = 2^(s-1), exact,
            // in one multiply while that factor is a bf16 (s <= 128), else in two
            const uint32_t s1 = sc < 128u ? sc : 128u;
            const uint32_t m1 = (s1 + 126u) << 7;
            const uint32_t mul = m1 | (m1 << 16);
            // 128-byte swizzle: 16-byte chunk j of row r sits at chunk j ^ (r & 7)
            unsigned char *row = slot + wr * 128 + (((hf * 4) ^ (wr & 4)) << 4);
            const int x3 = wr & 3;
            const uint32_t words[4] = {q0.x, q0.y, q0.z, q0.w};
            // (a scale above 2^1 is in no real checkpoint: one vote per chunk keeps the second
            // multiply out of the common path without a branch per lane)
            const bool two = __any_sync(0xffffffffu, sc > 128u);
            const uint32_t m2 = (sc > 128u ? sc - 1u : 127u) << 7, mul2 = m2 | (m2 << 16);
#pragma unroll
            for (int j = 0; j < 4; j++) {  // 8 elements (one packed word) -> one 16-byte chunk
              // the loader left the word as e0 e2 e4 e6 | e1 e3 e5 e7 (4 bits each, e0 lowest):
              // elements 2p and 2p + 1 are 16 bits apart
              const uint32_t w = words[j], w8 = w >> 8;
              uint4 o;
              o.x = bf16x2_mul(e2m1_pair_to_bf16x2_raw<true>(w & 0x000F000Fu), mul);
              o.y = bf16x2_mul(e2m1_pair_to_bf16x2_raw<false>(w & 0x00F000F0u), mul);
              o.z = bf16x2_mul(e2m1_pair_to_bf16x2_raw<true>(w8 & 0x000F000Fu), mul);
              o.w = bf16x2_mul(e2m1_pair_to_bf16x2_raw<false>(w8 & 0x00F000F0u), mul);
              if (two) {
                o.x = bf16x2_mul(o.x, mul2);
                o.y = bf16x2_mul(o.y, mul2);
                o.z = bf16x2_mul(o.z, mul2);
                o.w = bf16x2_mul(o.w, mul2);
              }
              *reinterpret_cast<uint4 *>(row + ((j ^ x3) << 4)) = o;
            }
          }
        }
        if (!TA) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&raw_empty[rs]);
          if (rank == 0)
            mbar_arrive(&full_bar[stage]);
          else
            mbar_arrive_cluster(&full_bar[stage], 0);
        }
      }
    }
  } else {
    using ST = PairStage<EPI>;
    const int q = warp & 3;            // TMEM lanes [32q, 32q+32)
    const int half = (warp - 2) >> 2;  // token chunks c with (c & 1) == half
    const int tg = ((warp - 2) & 3) * 32 + lane;  // thread index among the half's 4 warps
    const bool odd = (lane & 1) != 0;
    int acc = 0, buf = 0;
    uint32_t acc_phase = 0;
    for (int tile = first_tile; tile < total_tiles; tile += ncl) {
      int tt, wp;
      decode_tile(tile, w_pairs, tt_lo, &tt, &wp);
      const int e = g.mtile_expert[tt];
      const int tok0 = g.mtile_row0[tt];
      const int ntok = g.mtile_rows[tt];
      const int n_cta = wp * 256 + static_cast<int>(rank) * 128;  // first weight row of this CTA
      const int n_lane = n_cta + q * 32 + lane;
      const float bias_v = (g.bias != nullptr && n_lane < g.n_cols)
                               ? __ldg(g.bias + static_cast<size_t>(e) * g.n_cols + n_lane)
                               : 0.f;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) {
        set_status(g.status, kStatusWaitTimeoutEpilogue);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * kAccStride;
      const int n_chunks = (ntok + 31) >> 5;
      {
        for (int c = half; c < n_chunks; c += 2) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait32(r);
          unsigned char *tile_s = epi_stage + (half * 2 + buf) * ST::kTileBytes;
          if (EPI == kEpiSwiglu) {
            // lanes (2i, 2i+1) hold gate and up of feature i; each of the two takes
            // every other token
#pragma unroll
            for (int m = 0; m < 16; m++) {
              const float lo = __uint_as_float(r[2 * m]) + bias_v;
              const float hi = __uint_as_float(r[2 * m + 1]) + bias_v;
              const float own = odd ? hi : lo;
              const float send = odd ? lo : hi;
              const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
              const float a = swiglu_act(odd ? recv : own, odd ? own : recv, g.limit);
              const int j = 2 * m + (odd ? 1 : 0);
              *reinterpret_cast<bf16 *>(tile_s + j * ST::kPitch + q * 32 + (lane >> 1) * 2) =
                  __float2bfloat16_rn(a);
            }
          } else if (EPI == kEpiF32) {
            // lane = output column, register j = token: rows of 128 fp32 per CTA
#pragma unroll
            for (int j = 0; j < 32; j++)
              *reinterpret_cast<float *>(tile_s + j * ST::kPitch + q * 128 + lane * 4) =
                  __uint_as_float(r[j]) + bias_v;
          } else {
            const int jt = c * 32 + lane;
            const float w_lane = jt < ntok ? g.row_weight[tok0 + jt] : 0.f;
#pragma unroll
            for (int j = 0; j < 32; j++)
              r[j] = __float_as_uint((__uint_as_float(r[j]) + bias_v) *
                                     __shfl_sync(0xffffffffu, w_lane, j));
            // lanes (2i, 2i+1) hold columns (2i, 2i+1); each takes every other token
            // and stores both columns as one 32-bit word
#pragma unroll
            for (int m = 0; m < 16; m++) {
              const float own = __uint_as_float(odd ? r[2 * m + 1] : r[2 * m]);
              const float send = __uint_as_float(odd ? r[2 * m] : r[2 * m + 1]);
              const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
              const int j = 2 * m + (odd ? 1 : 0);
              *reinterpret_cast<uint32_t *>(tile_s + j * ST::kPitch + q * 64 + (lane >> 1) * 4) =
                  pack_bf16(odd ? recv : own, odd ? own : recv);
            }
          }
          // make the tile visible to the bulk-copy engine; the first warp of the half
          // also makes sure the copy that last read the other buffer is done before
          // anyone passes the barrier and starts to refill it
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          if (tg < 32) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          named_barrier_sync(1 + half, 128);
          // write out: one bulk copy per token row (a whole 128- / 256-byte segment)
          const int col0 = (EPI == kEpiSwiglu) ? (n_cta >> 1) : n_cta;
          if (tg < 32) {
            const int jt = c * 32 + tg;
            constexpr int kOutElem = (EPI == kEpiF32) ? 4 : 2;  // bytes per output element
            int bytes = (g.out_ld - col0) * kOutElem;
            bytes = bytes < ST::kRowBytes ? bytes : ST::kRowBytes;
            if (jt < ntok && bytes > 0) {
              unsigned char *dst =
                  (EPI == kEpiDown && g.row_dst != nullptr)
                      ? reinterpret_cast<unsigned char *>(g.row_dst[tok0 + jt]) +
                            static_cast<size_t>(col0) * kOutElem
                      : reinterpret_cast<unsigned char *>(g.out) +
                            (static_cast<size_t>(tok0 + jt) * g.out_ld + col0) * kOutElem;
              asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
                           "r"(smem_u32(tile_s + tg * ST::kPitch)), "r"(bytes)
                           : "memory");
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          buf ^= 1;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0)
          mbar_arrive(&tempty_bar[acc]);
        else
          mbar_arrive_cluster(&tempty_bar[acc], 0);
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    // the staging tiles must outlive the bulk copies that read them
    if (tg < 32) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) {
    }
  }
  cluster_barrier_all();  // neither CTA frees TMEM while the pair may still use it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <int EPI, int STAGES, bool MX, int TOKB, int RAWS, bool TA = false>
static cudaError_t launch_pair_stages(int num_sms, long long *launches, const CUtensorMap &tw,
                                      const CUtensorMap *tx, const GemmArgs &g,
                                      cudaStream_t stream, bool dependent = false) {
  constexpr int kbs = TA ? kTaKbs : 1;  // K blocks per ring stage
  const size_t smem = 1024 + STAGES * ((TA ? 0 : kPairOperandBytes) + kbs * TOKB * kTileK * 2) +
                      kPairBarrierBytes +
                      PairStage<EPI>::kTotalBytes +
                      (MX ? RAWS * kbs * kRawStageBytes : 0);
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_pair_kernel<EPI, STAGES, MX, TOKB, RAWS, TA>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(num_sms & ~1));
  cfg.blockDim = dim3(kPairThreads + (MX ? (dq_warps(STAGES) + 1) * 32 : 0));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 2 : 1;
  if (launches) ++*launches;
  return cudaLaunchKernelEx(&cfg, grouped_gemm_pair_kernel<EPI, STAGES, MX, TOKB, RAWS, TA>, tw,
                            tx[0], tx[1], tx[2], g);
}

template <int EPI>
// tx: the token-side tensor maps with boxes of 128, 32 and 8 rows
static cudaError_t launch_pair(gptoss_moe *h, const CUtensorMap &tw, const CUtensorMap *tx,
                               const GemmArgs &g, cudaStream_t stream) {
  const bool dep = h->opt_dependent_launch != 0;
  // MXFP4: four operand stages, one per group of four expanding warps; the packed weights wait
  // in the raw ring, which is what covers HBM latency (24 K blocks of 4.25 KB per CTA beside
  // the small token slots of decode-sized batches, 12 beside full-width ones).  Decode-sized
  // batches take the variant with three K blocks per stage and the expanded weights in TMEM
  // (18-30 % less time per layer at 64-1024 tokens than with one K block per stage and the
  // weights expanded into shared memory, which "mx_tmem" = 0 still selects).  Neither more
  // stages (six, with three groups alternating between two each; five with five groups)
  // nor the TMEM operand alone (2 %) changed the one-K-block form: its hand-shakes set the pace.
  if (h->cfg.weight_format == GPTOSS_WEIGHTS_MXFP4) {
    if (h->cur_tile_rows == 64) {
      if (h->opt_mx_tmem)
        return launch_pair_stages<EPI, 4, true, 32, 8, true>(h->num_sms, &h->launches, tx[0], tx,
                                                              g, stream, dep);
      return launch_pair_stages<EPI, 4, true, 32, 24>(h->num_sms, &h->launches, tx[0], tx, g,
                                                      stream, dep);
    }
    return launch_pair_stages<EPI, 4, true, 128, 12>(h->num_sms, &h->launches, tx[0], tx, g,
                                                     stream, dep);
  }
  return launch_pair_stages<EPI, 6, false, 128, 0>(h->num_sms, &h->launches, tw, tx, g, stream,
                                                      dep);
}

static GemmArgs pair_args(gptoss_moe *h, bool down, const LayerWeights &lw) {
  GemmArgs g;
  g.bias = down ? lw.b2 : lw.b1;
  g.out = down ? h->ys : h->hact;
  g.row_weight = down ? h->sorted_weight : nullptr;
  g.mtile_expert = h->mtile_expert;
  g.mtile_row0 = h->mtile_row0;
  g.mtile_rows = h->mtile_rows;
  g.num_mtiles = h->num_mtiles;
  g.k_dim = down ? h->IM : h->H;
  g.n_cols = down ? h->H : 2 * h->IM;
  g.out_ld = down ? h->H : h->IM;
  g.limit = h->cfg.swiglu_limit;
  g.status = h->status;
  g.wq = down ? lw.w2_blocks : lw.w1_blocks;
  g.l2_hints = h->opt_l2_hints;
  g.row_dst = (down && h->push_rows) ? h->row_dst : nullptr;
  return g;
}

cudaError_t launch_gate_up_pair(gptoss_moe *h, int layer, cudaStream_t stream, int part) {
  LayerWeights &lw = h->layers[layer];
  const CUtensorMap tx[3] = {h->tmap_xs, h->tmap_xs32, h->tmap_xs8};
  GemmArgs g = pair_args(h, false, lw);
  g.tile_part = part;
  g.tile_split = h->mtile_split;
  return launch_pair<kEpiSwiglu>(h, lw.tmap_w1_rows, tx, g, stream);
}

// A plain linear layer out[r, :] = (x[r, :] . W^T + bias) * row_weight[r] on the same kernel:
// one "expert" whose rows are all the rows of x, schedule and tensor maps supplied by the
// caller (tw: W [n_cols, k] in boxes of 128 rows; tx: x [rows, k] in boxes of 128, 32 and 8
// rows).
// f32_out: g.out addresses fp32 [rows, out_ld] (out_ld a multiple of 4), no row weight, bias
// optional; four operand stages make room for the wider output staging.
cudaError_t launch_linear_pair(int num_sms, const CUtensorMap &tw, const CUtensorMap *tx,
                               const GemmArgs &g, cudaStream_t stream, long long *launches,
                               bool f32_out) {
  if (f32_out)
    return launch_pair_stages<kEpiF32, 4, false, 128, 0>(num_sms, launches, tw, tx, g, stream);
  return launch_pair_stages<kEpiDown, 6, false, 128, 0>(num_sms, launches, tw, tx, g, stream);
}

cudaError_t launch_down_pair(gptoss_moe *h, int layer, cudaStream_t stream) {
  LayerWeights &lw = h->layers[layer];
  const CUtensorMap tx[3] = {h->tmap_h, h->tmap_h32, h->tmap_h8};
  return launch_pair<kEpiDown>(h, lw.tmap_w2_rows, tx, pair_args(h, true, lw), stream);
}

}  // namespace gptoss
