// Epilogue of the grouped GEMMs: TMEM accumulators -> bias -> activation or
// routing weight -> bf16 -> global memory.
//
// A warp owns 32 rows (its TMEM lane quarter) and a range of the tile's columns.
// Results are not stored straight from the thread that computed them (that would
// be one 16-byte piece in each of 32 different rows per instruction: half-filled
// sectors all over the place, which measurably slowed the main loop's own L2
// traffic); instead a pass of up to 128 output bytes per row is staged in a
// per-warp shared-memory tile and written out row-wise, 8 lanes per row, so a
// store instruction covers whole 128-byte row segments.
#pragma once
#include "common.cuh"

namespace gptoss {

// kEpiF32 (CTA-pair kernel only): out = acc (+ bias when given) as fp32, no row weight
enum { kEpiSwiglu = 0, kEpiDown = 1, kEpiF32 = 2 };

constexpr int kEpiPitch = 144;                  // 128 B of payload + 16 B: conflict-free
constexpr int kEpiStageBytes = 32 * kEpiPitch;  // per warp

struct GemmArgs {
  const float *bias;        // [El, n_cols]
  bf16 *out;                // hact [*, out_ld] or ys [*, out_ld]
  const float *row_weight;  // down only: routing weight per sorted row
  const int *mtile_expert, *mtile_row0, *mtile_rows, *num_mtiles;
  int k_dim;    // contraction length
  int n_cols;   // weight rows per expert
  int out_ld;   // leading dimension of out
  float limit;
  int *status;
  const uint8_t *wq = nullptr;  // MXFP4: tiled packed codes + scales of the weight operand
  // (CTA-pair kernel) 0 = every token tile; 1 / 2 = only the tiles before / from
  // *tile_split, so that a launch can start on the first experts while the rows of the
  // others are still on their way
  int tile_part = 0;
  const int *tile_split = nullptr;
  // (CTA-pair kernel) the loads carry L2 eviction hints: weights first out, token tiles last
  int l2_hints = 0;
  // (CTA-pair kernel, down epilogue) where row r of the output goes instead of out + r * out_ld:
  // the address of the row's first element, possibly in a peer GPU's memory
  const unsigned long long *row_dst = nullptr;
};

// gate * sigmoid(alpha * gate) * (up + 1) with the reference CPU path's clamps
// (run.cpp:711-724): gate from above only, up on both sides.
__device__ __forceinline__ float swiglu_act(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  const float s = __fdividef(1.0f, 1.0f + __expf(-1.702f * g));
  return g * s * (u + 1.0f);
}

// 16 accumulator columns n .. n+15 of one row -> bf16 pieces in the stage row.
// SwiGLU: 8 activations = one 16-byte piece; down: 16 values = two pieces.
template <int EPI>
__device__ __forceinline__ void epilogue_step16(const uint32_t *r, const float *bias, int n,
                                                int n_cols, float limit, float wrow,
                                                unsigned char *dst) {
  float v[16];
#pragma unroll
  for (int hlf = 0; hlf < 2; hlf++) {
    float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
    if (n + hlf * 8 + 8 <= n_cols) {
      b0 = __ldg(reinterpret_cast<const float4 *>(bias + n + hlf * 8));
      b1 = __ldg(reinterpret_cast<const float4 *>(bias + n + hlf * 8 + 4));
    }
    v[hlf * 8 + 0] = __uint_as_float(r[hlf * 8 + 0]) + b0.x;
    v[hlf * 8 + 1] = __uint_as_float(r[hlf * 8 + 1]) + b0.y;
    v[hlf * 8 + 2] = __uint_as_float(r[hlf * 8 + 2]) + b0.z;
    v[hlf * 8 + 3] = __uint_as_float(r[hlf * 8 + 3]) + b0.w;
    v[hlf * 8 + 4] = __uint_as_float(r[hlf * 8 + 4]) + b1.x;
    v[hlf * 8 + 5] = __uint_as_float(r[hlf * 8 + 5]) + b1.y;
    v[hlf * 8 + 6] = __uint_as_float(r[hlf * 8 + 6]) + b1.z;
    v[hlf * 8 + 7] = __uint_as_float(r[hlf * 8 + 7]) + b1.w;
  }
  if (EPI == kEpiSwiglu) {
    uint4 o;
    o.x = pack_bf16(swiglu_act(v[0], v[1], limit), swiglu_act(v[2], v[3], limit));
    o.y = pack_bf16(swiglu_act(v[4], v[5], limit), swiglu_act(v[6], v[7], limit));
    o.z = pack_bf16(swiglu_act(v[8], v[9], limit), swiglu_act(v[10], v[11], limit));
    o.w = pack_bf16(swiglu_act(v[12], v[13], limit), swiglu_act(v[14], v[15], limit));
    *reinterpret_cast<uint4 *>(dst) = o;
  } else {
    uint4 o;
    o.x = pack_bf16(v[0] * wrow, v[1] * wrow);
    o.y = pack_bf16(v[2] * wrow, v[3] * wrow);
    o.z = pack_bf16(v[4] * wrow, v[5] * wrow);
    o.w = pack_bf16(v[6] * wrow, v[7] * wrow);
    *reinterpret_cast<uint4 *>(dst) = o;
    o.x = pack_bf16(v[8] * wrow, v[9] * wrow);
    o.y = pack_bf16(v[10] * wrow, v[11] * wrow);
    o.z = pack_bf16(v[12] * wrow, v[13] * wrow);
    o.w = pack_bf16(v[14] * wrow, v[15] * wrow);
    *reinterpret_cast<uint4 *>(dst + 16) = o;
  }
}

// One pass: PC accumulator columns (multiple of 16, <= 128 for SwiGLU, <= 64 for
// down) starting at TMEM address taddr / expert column n0; rows row0+q*32 ..,
// `rows_left` of which exist.  stage = this warp's [32][kEpiPitch] tile.
template <int EPI, int PC>
__device__ __forceinline__ void epilogue_pass(uint32_t taddr, int n0, const float *bias,
                                              int row_base, int rows_left, int lane, float wrow,
                                              const GemmArgs &g, unsigned char *stage) {
  constexpr int kOutBytesPer16 = (EPI == kEpiSwiglu) ? 16 : 32;
  constexpr int kFull = PC / 32;
  constexpr bool kTail = (PC % 32) != 0;
  unsigned char *my = stage + lane * kEpiPitch;
  uint32_t ra[32], rb[32];
  if (kFull > 0) {
    tmem_ld32(taddr, ra);
  } else {
    tmem_ld16(taddr, *reinterpret_cast<uint32_t(*)[16]>(ra));
  }
  tmem_ld_wait32(ra);
#pragma unroll
  for (int c = 0; c < kFull; c += 2) {
    if (c + 1 < kFull) {
      tmem_ld32(taddr + (c + 1) * 32, rb);
    } else if (kTail) {
      tmem_ld16(taddr + kFull * 32, *reinterpret_cast<uint32_t(*)[16]>(rb));
    }
    epilogue_step16<EPI>(ra, bias, n0 + c * 32, g.n_cols, g.limit, wrow,
                         my + (c * 2) * kOutBytesPer16);
    epilogue_step16<EPI>(ra + 16, bias, n0 + c * 32 + 16, g.n_cols, g.limit, wrow,
                         my + (c * 2 + 1) * kOutBytesPer16);
    if (c + 1 < kFull || kTail) tmem_ld_wait32(rb);
    if (c + 1 < kFull) {
      if (c + 2 < kFull) {
        tmem_ld32(taddr + (c + 2) * 32, ra);
      } else if (kTail) {
        tmem_ld16(taddr + kFull * 32, *reinterpret_cast<uint32_t(*)[16]>(ra));
      }
      epilogue_step16<EPI>(rb, bias, n0 + (c + 1) * 32, g.n_cols, g.limit, wrow,
                           my + ((c + 1) * 2) * kOutBytesPer16);
      epilogue_step16<EPI>(rb + 16, bias, n0 + (c + 1) * 32 + 16, g.n_cols, g.limit, wrow,
                           my + ((c + 1) * 2 + 1) * kOutBytesPer16);
      if (c + 2 < kFull || kTail) tmem_ld_wait32(ra);
    }
  }
  if (kTail)
    epilogue_step16<EPI>((kFull & 1) ? rb : ra, bias, n0 + kFull * 32, g.n_cols, g.limit, wrow,
                         my + (kFull * 2) * kOutBytesPer16);
  __syncwarp();
  // write out: kLanes lanes per row, each one 16-byte piece
  constexpr int kRowBytes = PC / 16 * kOutBytesPer16;  // <= 128
  constexpr int kLanes = kRowBytes / 16;
  constexpr int kRowsPerInstr = 32 / kLanes;
  const int sub = lane / kLanes, piece = lane - sub * kLanes;
  const int out_col0 = (EPI == kEpiSwiglu) ? (n0 >> 1) : n0;
  const bool piece_ok = sub < kRowsPerInstr && out_col0 + piece * 8 + 8 <= g.out_ld;
#pragma unroll
  for (int r0 = 0; r0 < 32; r0 += kRowsPerInstr) {
    const int r = r0 + sub;
    if (piece_ok && r < 32 && r < rows_left) {
      const uint4 v = *reinterpret_cast<const uint4 *>(stage + r * kEpiPitch + piece * 16);
      // streaming store: the output is read once by the next kernel and must not
      // push the weight and activation tiles this kernel re-reads out of L2
      __stcs(reinterpret_cast<uint4 *>(g.out + static_cast<size_t>(row_base + r) * g.out_ld +
                                       out_col0 + piece * 8),
             v);
    }
  }
  __syncwarp();
}

// NC accumulator columns (multiple of 16) of the warp's 32 rows, in passes.
template <int EPI, int NC>
__device__ __forceinline__ void epilogue_cols(uint32_t taddr, int n0, int e, int row_base,
                                              int rows_left, int lane, float wrow,
                                              const GemmArgs &g, unsigned char *stage) {
  constexpr int kPass = (EPI == kEpiSwiglu) ? 128 : 64;
  const float *bias = g.bias + static_cast<size_t>(e) * g.n_cols;
  constexpr int kPasses = NC / kPass;
  constexpr int kRest = NC % kPass;
#pragma unroll
  for (int p = 0; p < kPasses; p++)
    epilogue_pass<EPI, kPass>(taddr + p * kPass, n0 + p * kPass, bias, row_base, rows_left, lane,
                              wrow, g, stage);
  if (kRest > 0)
    epilogue_pass<EPI, (kRest > 0 ? kRest : 16)>(taddr + kPasses * kPass, n0 + kPasses * kPass,
                                                 bias, row_base, rows_left, lane, wrow, g, stage);
}

}  // namespace gptoss
