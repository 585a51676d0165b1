// lt2exp:  out[r,s,k] = ma[r,k] + mb[r,k] + log( sum_{i,j} w[r,s,i,j] * exp(a[r,i,k]-ma[r,k]) * exp(b[r,j,k]-mb[r,k]) )
//
// Replaces the reference's Triton kernels _ker_lt2exp_unsplit / _ker_lt2exp_split
// (triturus/lt2exp.py:227-357, 365-506) with one persistent, warp-specialised sm_100a kernel.
// As a GEMM: D[M = s, N = k] = W[M, Kc = (i,j)] * P[Kc, N] with the Khatri-Rao operand
// P[(i,j), k] = exp(a[i,k]-ma[k]) * exp(b[j,k]-mb[k]), which is generated tile by tile in shared memory and
// never written to HBM (the reference's torch baseline materialises it, baselines/lt2exp.py:21-22, and its
// Triton kernels recompute both exps for every (i,j) pair, triturus/lt2exp.py:337-338).
//
// One k-block of the contraction is one i and 32 consecutive j (a 128-byte row segment of w), fetched by a
// 4-D TMA box {32 j, 1 i, 128 s, 1 r} with the 128-byte swizzle; j past J is zero-filled.  k-blocks run with
// the j-chunk outermost so a transform thread keeps its 32 exp(b - mb) values in registers for I k-blocks
// and needs one exp(a - ma) per k-block, prefetched from global memory eight k-blocks ahead.
//
//   warp 0      TMA producer (w tiles).
//   warp 1      TMEM allocation; one lane issues tcgen05.mma.kind::tf32 and commits.
//   warps 4-7   epilogue: out = (ma + mb) + log(acc).
//   warps 8+    transform: column maxima of a and b (-inf safe), then the P operand of every k-block.
//               The NTT / BN thread groups take alternate k-blocks.
//
// Contraction split.  A shape with few output tiles (small batch, S and K) would leave most SMs idle while
// each busy one walks the whole (i, j) range, and a tile count that is not a multiple of the SM count leaves
// the last wave partly empty.  The launcher can therefore cut the contraction of every tile into nsplit equal
// slices, one work item each, or (stream) run all full waves of tiles whole and share only the tiles of the
// last, partly filled wave among all CTAs.  All parts of a tile use the same stabilisers (the
// column maxima are taken over the full I and J), so their accumulators add linearly: in these modes the
// epilogue adds its raw accumulator into the zero-filled output with red.global.add and
// lt2exp_finish_kernel then turns the sums into (ma + mb) + log(sum) in place.
//
// Accumulator promotion (3xTF32 always; plain TF32 in the PROMOTE instances the launcher picks for contractions
// of more than 32 K terms).  The tensor core adds into its fp32 accumulator with truncation, so a
// sum of positive terms drifts low by about half an ulp per MMA: ~3e-8 relative per 8 contraction terms,
// 1e-4 after 32 K terms and 2.5e-3 after 256 K, far more than the 3xTF32 operand error.  In 3xTF32 mode
// the MMA warp therefore starts a fresh TMEM accumulator every CHUNK k-blocks and the epilogue warps, idle
// during the main loop, add each finished chunk into a master copy kept in a further TMEM region with
// round-to-nearest fp32 adds (tcgen05.ld, add, tcgen05.st).  Plain TF32 on shorter contractions keeps one chunk
// per work item: the drift stays below 3e-4 there, well inside the 2e-3 tolerance of that mode.
#pragma once

#include "ptx.cuh"

namespace tb200 {

struct Lt2expParams {
  const float* a;  // [R, I, K]
  const float* b;  // [R, J, K]
  float* out;      // [R, S, K]
  int64_t a_s0, a_s1, b_s0, b_s1;  // element strides of the batch and row dimensions
  int64_t a_s2 = 1, b_s2 = 1;      // ... and along k (any value; the 16-byte loads of vec_ab need 1)
  int64_t out_s0, out_s1;
  int R, S, I, J, K;
  int tiles_m, tiles_n, num_tiles;
  int nsplit;     // equal slices of the contraction per tile (1: whole tiles)
  int stream;     // 1: whole waves of tiles, then the tiles of the last wave shared among all CTAs (see LtWork)
  int num_items;  // num_tiles * nsplit (not used when stream == 1)
  int lw_first, lw_parts, lw_main;  // stream == 1: first tile of the last wave and how it is shared (see LtWork)
  // stream == 1 with scratch memory (both non-null): a tile that several CTAs share is completed without
  // atomics.  Every part but the first parks its raw partial sums in a slot of `park`
  // ([slot][MT * BN / 32 chunks][8 column quads][128 rows][4] floats: the 32 lanes of a store write 512
  // consecutive bytes) and then raises park_flags[slot] (zeroed by the launcher)
  // by one per epilogue warp; the CTA with the first part adds the parked sums to its own, in slot order, and
  // writes the finished results.
  float* park;
  int* park_flags;
  int vec_ab;            // a and b allow 16-byte loads along k (alignment, strides and K multiples of 4)
  int* status;
  // Chains of layers (all optional, contiguous [R, K]): column maxima of a and of b supplied by the caller
  // (both or neither; clamped when read), which replace the scan of a and b; and max_s out[r,s,k], which the
  // epilogue (or, for a split contraction, the log pass) folds into out_max, which the launcher fills with
  // -inf first.
  const float* ma_in;
  const float* mb_in;
  float* out_max;
};

// One work item: the k-blocks [kb_lo, kb_hi) of output tile `tile`.  k-block index = jc * I + i, so a range
// is whole rows of the (jc, i) grid plus a partial first and last row.
// park_slot >= 0: the item is not the first part of its tile; with scratch memory its raw sums are parked there.
// ncollect > 0: the item is the first part of a shared tile and completes it from the slots slot0 .. slot0 + ncollect - 1.
struct LtItem {
  int tile, kb_lo, kb_hi;
  int park_slot, slot0, ncollect;
};

// The work items of one CTA, in the order every role of the CTA walks them.
//  * stream == 0: item q = tile * nsplit + slice, slices of equal length, items taken round robin over the CTAs.
//  * stream == 1 ("whole waves, last wave shared out"): with G CTAs, the first (W - 1) * G tiles run as whole
//    tiles, round robin, exactly as without any split, so CTAs that read the same rows of w do so at the same
//    time and the rows cross HBM once.  (Cutting the k-blocks of all tiles into G equal contiguous ranges
//    balances as well but puts the CTAs that share rows of w at different offsets: measured 45 % slower on
//    R = 8 and R = 32 entries of 256 x 128 x 128 x 4096 because w then streams from HBM for every column tile.)
//    The `rem` tiles of the last wave are shared among all G CTAs:
//      rem <= G / 2:  every tile is cut into P = floor(G / rem) equal parts, part j of tile t on CTA t + j * rem;
//      rem >  G / 2:  CTA t < rem takes the first `lw_main` k-blocks of tile t, and each of the G - rem other
//                     CTAs takes the remaining k-blocks ("tails") of tiles u, u + (G - rem), ...; lw_main is
//                     chosen by the launcher so that a CTA with the most tails is busy as long as a main part.
//    The first part of a tile completes it (LtItem::ncollect), the other parts are parked or added.
struct LtWork {
  int q, nq, step;
  int kb_tile, nsplit, stream;
  int lw_first, lw_rem, lw_parts, lw_main;  // last wave: first tile, tiles, parts per tile (0: mains and tails), main length
  int phase, tail_next;                     // stream: 0 = whole waves, 1 = last wave, 2 = done
  __device__ LtWork(const Lt2expParams& p, int kb_tile_) {
    kb_tile = kb_tile_;
    nsplit = p.nsplit;
    stream = p.stream;
    q = blockIdx.x;
    nq = stream ? p.lw_first : p.num_items;
    step = gridDim.x;
    lw_first = p.lw_first;
    lw_rem = p.num_tiles - p.lw_first;
    lw_parts = p.lw_parts;
    lw_main = p.lw_main;
    phase = 0;
    tail_next = static_cast<int>(blockIdx.x) - lw_rem;  // (mains and tails) first tail of a helper CTA
  }
  __device__ bool next(LtItem& w) {
    w.park_slot = -1;
    w.slot0 = 0;
    w.ncollect = 0;
    if (!stream) {
      if (q >= nq) return false;
      w.tile = q / nsplit;
      const int sl = q - w.tile * nsplit;
      w.kb_lo = static_cast<int>(static_cast<int64_t>(sl) * kb_tile / nsplit);
      w.kb_hi = static_cast<int>(static_cast<int64_t>(sl + 1) * kb_tile / nsplit);
      q += step;
      return true;
    }
    if (phase == 0) {
      if (q < nq) {  // whole tiles of the full waves
        w.tile = q;
        w.kb_lo = 0;
        w.kb_hi = kb_tile;
        q += step;
        return true;
      }
      phase = 1;
    }
    if (phase != 1) return false;
    const int c = blockIdx.x;
    if (lw_parts > 0) {
      // equal parts: part j of tile t on CTA t + j * rem
      phase = 2;
      const int j = c / lw_rem, t = c - j * lw_rem;
      if (j >= lw_parts) return false;
      w.tile = lw_first + t;
      w.kb_lo = static_cast<int>(static_cast<int64_t>(j) * kb_tile / lw_parts);
      w.kb_hi = static_cast<int>(static_cast<int64_t>(j + 1) * kb_tile / lw_parts);
      if (lw_parts > 1) {
        if (j == 0) {
          w.slot0 = t * (lw_parts - 1);
          w.ncollect = lw_parts - 1;
        } else {
          w.park_slot = t * (lw_parts - 1) + (j - 1);
        }
      }
      return true;
    }
    if (c < lw_rem) {
      // main part of tile c
      phase = 2;
      w.tile = lw_first + c;
      w.kb_lo = 0;
      w.kb_hi = lw_main;
      w.slot0 = c;
      w.ncollect = lw_main < kb_tile ? 1 : 0;
      return true;
    }
    // tails of tiles u, u + (G - rem), ...
    if (tail_next >= lw_rem || lw_main >= kb_tile) {
      phase = 2;
      return false;
    }
    w.tile = lw_first + tail_next;
    w.kb_lo = lw_main;
    w.kb_hi = kb_tile;
    w.park_slot = tail_next;
    tail_next += static_cast<int>(gridDim.x) - lw_rem;
    return true;
  }
};

// Rows i of j-chunk jc that belong to the item: [lt_row_lo, lt_row_hi).
__device__ __forceinline__ int lt_row_lo(const LtItem& w, int jc, int I) {
  const int lo = w.kb_lo - jc * I;
  return lo > 0 ? lo : 0;
}
__device__ __forceinline__ int lt_row_hi(const LtItem& w, int jc, int I) {
  const int hi = w.kb_hi - jc * I;
  return hi < I ? hi : I;
}

template <int BN_, int MT_, int PREC_, int NS_, int NTW_, bool PROMOTE_ = (PREC_ != 0)>
struct Lt2expCfg {
  static constexpr int BM = 128, BK = 32;
  static constexpr int BN = BN_, MT = MT_, PREC = PREC_, NS = NS_, NTW = NTW_;
  static constexpr int NCOPY = PREC ? 2 : 1;
  static constexpr int A_TILE = BM * BK * 4;
  static constexpr int B_TILE = BN * BK * 4;
  static constexpr int STAGE = NCOPY * (MT * A_TILE + B_TILE);
  static constexpr int ACC_COLS = MT * BN;
  static constexpr bool PROMOTE = PROMOTE_;
  // k-blocks (of 32 terms) accumulated by the tensor core before a promotion: 1 K terms keep the drift near
  // 1e-5 for 3xTF32; plain TF32 (2e-3 budget, operand rounding ~1e-3) promotes every 4 K terms (~6e-5).
  static constexpr int CHUNK = PREC ? 32 : 128;
  // Accumulator buffers the MMA warp rotates through, and the master copy behind them when promoting.
  static constexpr int NBUF = PROMOTE ? ((3 * ACC_COLS <= 512) ? 2 : 1) : ((2 * ACC_COLS <= 512) ? 2 : 1);
  static constexpr int MASTER_COL = NBUF * ACC_COLS;
  static constexpr int TMEM_USED = (NBUF + (PROMOTE ? 1 : 0)) * ACC_COLS;
  static constexpr int TMEM_COLS = (TMEM_USED <= 128) ? 128 : (TMEM_USED <= 256 ? 256 : 512);
  static constexpr int NTHREADS = (8 + NTW) * 32;
  static constexpr int NTT = NTW * 32;
  static constexpr int NGROUPS = NTT / BN;      // transform thread groups taking alternate k-blocks
  static constexpr int GROUP_WARPS = BN / 32;
  // Column maxima are taken cooperatively: NTT threads = CQ column quads x RG row groups (16-byte loads).
  static constexpr int CQ = BN / 4;
  static constexpr int RG = NTT / CQ;
  static constexpr int MPART = 2 * RG * BN;  // floats per slot: partial maxima of a and of b
  static constexpr int NBAR = 3 * NS + 7;
  static constexpr int SMEM_BYTES = 1024 + NS * STAGE + 2 * BN * 4 + 2 * MPART * 4 + NBAR * 8 + 64;
  static_assert(NTT % CQ == 0 && RG >= NGROUPS, "column-maximum thread mapping");
  static_assert(NTT % BN == 0 && NGROUPS >= 1, "transform thread mapping");
  static_assert(TMEM_USED <= 512, "TMEM capacity");
  static_assert(SMEM_BYTES <= 232448, "shared memory capacity");
};

// Running maximum of four adjacent columns over rows first, first + step, ... < rows, sixteen 16-byte loads
// in flight (the scan is a chain of memory round trips: fewer, wider rounds).  `quad` points at row 0 of the
// four columns.
__device__ __forceinline__ float4 quad_column_max(const float* quad, int64_t stride, int rows, int first, int step) {
  float4 m = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
  int i = first;
  constexpr int INFLIGHT = 16;
  const float4 ninf = m;
  for (; i < rows; i += INFLIGHT * step) {
    float4 v[INFLIGHT];
#pragma unroll
    for (int x = 0; x < INFLIGHT; ++x) {
      const int row = i + x * step;
      v[x] = ninf;  // rows past the end do not change the maximum
      if (row < rows) v[x] = __ldg(reinterpret_cast<const float4*>(quad + static_cast<int64_t>(row) * stride));
    }
#pragma unroll
    for (int x = 0; x < INFLIGHT; ++x) {
      m.x = fmaxf(m.x, v[x].x);
      m.y = fmaxf(m.y, v[x].y);
      m.z = fmaxf(m.z, v[x].z);
      m.w = fmaxf(m.w, v[x].w);
    }
  }
  return m;
}

// Same for one column (the fallback when 16-byte loads are not possible).
__device__ __forceinline__ float strided_column_max(const float* col, int64_t stride, int rows, int first, int step) {
  float m = -INFINITY;
  int i = first;
  for (; i + 15 * step < rows; i += 16 * step) {
    float v[16];
#pragma unroll
    for (int x = 0; x < 16; ++x) v[x] = __ldg(col + static_cast<int64_t>(i + x * step) * stride);
#pragma unroll
    for (int x = 0; x < 16; ++x) m = fmaxf(m, v[x]);
  }
  for (; i < rows; i += step) m = fmaxf(m, __ldg(col + static_cast<int64_t>(i) * stride));
  return m;
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
lt2exp_kernel(const __grid_constant__ CUtensorMap tmap_w, const Lt2expParams p) {
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, MT = Cfg::MT, NS = Cfg::NS;
  constexpr int PREC = Cfg::PREC;
  constexpr int PF = 8;  // prefetch distance (own k-blocks) for the a values

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  float* msum = reinterpret_cast<float*>(smem + NS * Cfg::STAGE);  // [2][BN]: ma + mb of the tile's columns
  float* mpart = msum + 2 * BN;  // [2][2][RG][BN] partial column maxima (slot, a|b, row group, column)
  uint64_t* bars = reinterpret_cast<uint64_t*>(mpart + 2 * Cfg::MPART);
  uint64_t* a_full = bars;               // [NS] w tiles landed
  uint64_t* b_full = bars + NS;          // [NS] P operand (and w split) written
  uint64_t* opnd_empty = bars + 2 * NS;  // [NS] MMAs reading the stage retired
  uint64_t* acc_full = bars + 3 * NS;    // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint64_t* msum_empty = acc_empty + 2;  // [2] epilogue finished reading msum[slot]
  uint64_t* mx_bar = msum_empty + 2;     // [1] every transform warp published its partial maxima
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mx_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AbortCtl ctl{abort_flag, p.status};

  auto a_tile = [&](int s, int c, int t) -> uint8_t* {
    return stage_base + s * Cfg::STAGE + (c * MT + t) * Cfg::A_TILE;
  };
  auto b_tile = [&](int s, int c) -> uint8_t* {
    return stage_base + s * Cfg::STAGE + Cfg::NCOPY * MT * Cfg::A_TILE + c * Cfg::B_TILE;
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < NS; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&b_full[s], Cfg::GROUP_WARPS);
      mbar_init(&opnd_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 4);
      mbar_init(&msum_empty[s], 4);
    }
    mbar_init(mx_bar, Cfg::NTW);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int JC = (p.J + BK - 1) / BK;  // j-chunks; the k-blocks of a work item are (jc, i), i fastest
  const int KBT = JC * p.I;            // k-blocks per output tile
  const bool parking = p.stream != 0 && p.park != nullptr;  // shared tiles are completed through scratch memory
  const bool split_mode = (p.nsplit > 1 || p.stream != 0) && !parking;  // partial sums are added into the zero-filled output

  // Output tile -> (r, n0 = first column, s0 = first row).
  auto decode = [&](int tile, int& r, int& n0, int& s0) {
    const int tm = tile % p.tiles_m;
    const int rest = tile / p.tiles_m;
    const int tn = rest % p.tiles_n;
    r = rest / p.tiles_n;
    n0 = tn * BN;
    s0 = tm * (BM * MT);
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      LtWork work(p, KBT);
      for (LtItem w; ok && work.next(w);) {
        int r, n0, s0;
        decode(w.tile, r, n0, s0);
        for (int jc = w.kb_lo / p.I; ok && jc * p.I < w.kb_hi; ++jc) {
          const int i_hi = lt_row_hi(w, jc, p.I);
          for (int i = lt_row_lo(w, jc, p.I); i < i_hi; ++i, ++it) {
            const int s = it % NS;
            const uint32_t ph = (it / NS) & 1;
            if (!(ok = mbar_wait(&opnd_empty[s], ph ^ 1, ctl, STATUS_TIMEOUT_PRODUCER))) break;
            mbar_arrive_expect_tx(&a_full[s], MT * Cfg::A_TILE);
#pragma unroll
            for (int t = 0; t < MT; ++t)
              tma_load_4d(a_tile(s, 0, t), &tmap_w, &a_full[s], jc * BK, i, s0 + t * BM, r);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(BM, BN);
      uint32_t it = 0, ccount = 0;  // k-blocks and accumulation chunks issued so far
      bool ok = true;
      LtWork work(p, KBT);
      for (LtItem w; ok && work.next(w);) {
        const int KB = w.kb_hi - w.kb_lo;
        const int nch = Cfg::PROMOTE ? (KB + Cfg::CHUNK - 1) / Cfg::CHUNK : 1;
        int kb = 0;
        for (int ch = 0; ok && ch < nch; ++ch, ++ccount) {
          const int buf = ccount % Cfg::NBUF;
          const uint32_t aph = (ccount / Cfg::NBUF) & 1;
          if (!(ok = mbar_wait(&acc_empty[buf], aph ^ 1, ctl, STATUS_TIMEOUT_MMA))) break;
          tc_fence_after_sync();
          const int kb0 = kb;
          const int kb_end = Cfg::PROMOTE ? min(KB, kb0 + Cfg::CHUNK) : KB;
          for (; kb < kb_end; ++kb, ++it) {
            const int s = it % NS;
            const uint32_t ph = (it / NS) & 1;
            if (!(ok = mbar_wait(&a_full[s], ph, ctl, STATUS_TIMEOUT_MMA))) break;
            if (!(ok = mbar_wait(&b_full[s], ph, ctl, STATUS_TIMEOUT_MMA))) break;
            tc_fence_after_sync();
            const uint64_t db_hi = umma_desc_k_sw128(smem_u32(b_tile(s, 0)));
            const uint64_t db_lo = PREC ? umma_desc_k_sw128(smem_u32(b_tile(s, 1))) : 0;
#pragma unroll
            for (int t = 0; t < MT; ++t) {
              const uint32_t d = tmem_base + buf * Cfg::ACC_COLS + t * BN;
              const uint64_t da_hi = umma_desc_k_sw128(smem_u32(a_tile(s, 0, t)));
              const uint64_t da_lo = PREC ? umma_desc_k_sw128(smem_u32(a_tile(s, 1, t))) : 0;
#pragma unroll
              for (int ks = 0; ks < BK / 8; ++ks) {
                const uint32_t acc = (kb > kb0 || ks > 0) ? 1u : 0u;
                if (PREC) {
                  umma_tf32_ss(d, da_hi + 2 * ks, db_lo + 2 * ks, idesc, acc);
                  umma_tf32_ss(d, da_lo + 2 * ks, db_hi + 2 * ks, idesc, 1u);
                  umma_tf32_ss(d, da_hi + 2 * ks, db_hi + 2 * ks, idesc, 1u);
                } else {
                  umma_tf32_ss(d, da_hi + 2 * ks, db_hi + 2 * ks, idesc, acc);
                }
              }
            }
            umma_commit(&opnd_empty[s]);
          }
          if (ok) umma_commit(&acc_full[buf]);
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const bool vec_ok = ((p.K & 3) == 0) && ((p.out_s1 & 3) == 0) && ((p.out_s0 & 3) == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    uint32_t tcount = 0, ccount = 0;
    bool ok = true;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    LtWork work(p, KBT);
    for (LtItem w; ok && work.next(w); ++tcount) {
      int r, n0, s0;
      decode(w.tile, r, n0, s0);
      const int KB = w.kb_hi - w.kb_lo;
      const int nch = Cfg::PROMOTE ? (KB + Cfg::CHUNK - 1) / Cfg::CHUNK : 1;
      const int slot = tcount & 1;
      // Stream mode with scratch memory: a part that is not the first of its tile parks its sums; the first part
      // of a shared tile collects them.
      const bool park_it = parking && w.park_slot >= 0;
      const bool collect = parking && w.ncollect > 0;
      if (collect) {
        // The other parts run at the same time on other CTAs and end about when this one does.
        for (int cc = 0; ok && cc < w.ncollect; ++cc) {
          const long long t0 = clock64();
          while (ld_acquire_gpu(p.park_flags + w.slot0 + cc) < 4) {
            if (*ctl.flag || clock64() - t0 > WAIT_LIMIT_CYCLES) {
              raise_abort(ctl, STATUS_TIMEOUT_EPILOGUE);
              ok = false;
              break;
            }
          }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      constexpr int PARK_TILE = MT * BN * BM;  // floats per parked tile
      for (int ch = 0; ok && ch < nch; ++ch, ++ccount) {
        const int buf = ccount % Cfg::NBUF;
        const uint32_t aph = (ccount / Cfg::NBUF) & 1;
        const bool first = ch == 0, last = ch == nch - 1;
        if (!(ok = mbar_wait_warp(&acc_full[buf], aph, ctl, STATUS_TIMEOUT_EPILOGUE))) break;
        tc_fence_after_sync();
#pragma unroll 1
        for (int t = 0; t < MT; ++t) {
          if (s0 + t * BM >= p.S) break;
          const int row = s0 + t * BM + q * 32 + lane;
          float* out_row = p.out + static_cast<int64_t>(r) * p.out_s0 + static_cast<int64_t>(row) * p.out_s1;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            const int k0 = n0 + c * 32;
            if (k0 >= p.K) break;
            uint32_t v[32];
            tmem_ld_32x32(lane_base + buf * Cfg::ACC_COLS + t * BN + c * 32, v);
            if (Cfg::PROMOTE) {
              // Chunks after the first are added to the master copy; all but the last are stored back.
              const uint32_t master = lane_base + Cfg::MASTER_COL + t * BN + c * 32;
              if (!first) {
                uint32_t mv[32];
                tmem_ld_32x32(master, mv);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e)
                  v[e] = __float_as_uint(__fadd_rn(__uint_as_float(v[e]), __uint_as_float(mv[e])));
              }
              if (!last) {
                tmem_ld_wait();
                tmem_st_32x32(master, v);
                continue;
              }
            }
            if (park_it) {
              // Raw sums of this (row block, column chunk) to the part's slot, four columns of 32 rows per store.
              tmem_ld_wait();
              float4* dst = reinterpret_cast<float4*>(p.park + static_cast<int64_t>(w.park_slot) * PARK_TILE +
                                                      static_cast<int64_t>(t * (BN / 32) + c) * BM * 32) +
                            q * 32 + lane;
#pragma unroll
              for (int g = 0; g < 8; ++g)
                dst[g * BM] = make_float4(__uint_as_float(v[g * 4]), __uint_as_float(v[g * 4 + 1]), __uint_as_float(v[g * 4 + 2]),
                                     __uint_as_float(v[g * 4 + 3]));
              continue;
            }
            if (collect) {
              tmem_ld_wait();
              for (int cc = 0; cc < w.ncollect; ++cc) {
                const float4* src = reinterpret_cast<const float4*>(
                                        p.park + static_cast<int64_t>(w.slot0 + cc) * PARK_TILE +
                                        static_cast<int64_t>(t * (BN / 32) + c) * BM * 32) +
                                    q * 32 + lane;
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                  const float4 x = __ldcg(src + g * BM);  // written during this launch: not through the read-only path
                  v[g * 4 + 0] = __float_as_uint(__uint_as_float(v[g * 4 + 0]) + x.x);
                  v[g * 4 + 1] = __float_as_uint(__uint_as_float(v[g * 4 + 1]) + x.y);
                  v[g * 4 + 2] = __float_as_uint(__uint_as_float(v[g * 4 + 2]) + x.z);
                  v[g * 4 + 3] = __float_as_uint(__uint_as_float(v[g * 4 + 3]) + x.w);
                }
              }
            }
            if (split_mode) {
              // Slice of a split contraction: add the raw accumulator into the zero-filled output.
              tmem_ld_wait();
              if (row < p.S) {
                if (vec_ok) {
#pragma unroll
                  for (int g = 0; g < 8; ++g) {
                    if (k0 + g * 4 < p.K)
                      red_add_f32x4(out_row + k0 + g * 4, __uint_as_float(v[g * 4]), __uint_as_float(v[g * 4 + 1]),
                                    __uint_as_float(v[g * 4 + 2]), __uint_as_float(v[g * 4 + 3]));
                  }
                } else {
#pragma unroll
                  for (int e = 0; e < 32; ++e) {
                    if (k0 + e < p.K) atomicAdd(out_row + k0 + e, __uint_as_float(v[e]));
                  }
                }
              }
              continue;
            }
            const float m_lane = msum[slot * BN + c * 32 + lane];
            tmem_ld_wait();
            float o[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float m_e = __shfl_sync(0xffffffffu, m_lane, e);
              const float acc = __uint_as_float(v[e]);
              o[e] = m_e + (PREC ? logf(acc) : lg2_approx(acc) * LN2_F);
            }
            if (row < p.S) {
              if (vec_ok) {
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                  if (k0 + g * 4 < p.K) {
                    *reinterpret_cast<float4*>(out_row + k0 + g * 4) =
                        make_float4(o[g * 4], o[g * 4 + 1], o[g * 4 + 2], o[g * 4 + 3]);
                  }
                }
              } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                  if (k0 + e < p.K) out_row[k0 + e] = o[e];
                }
              }
            }
            if (p.out_max != nullptr) {
              // Column maxima of this 32 x 32 block for the next layer.  A tile of this kernel is hundreds of
              // k-blocks long, so one reduction per block and warp straight into global memory is negligible.
              const float cmx = block_colmax_to_lanes(o, row < p.S, lane);
              if (k0 + lane < p.K) red_max_f32(p.out_max + static_cast<int64_t>(r) * p.K + k0 + lane, cmx);
            }
          }
        }
        if (Cfg::PROMOTE && !last) tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&acc_empty[buf]);
          if (last) mbar_arrive(&msum_empty[slot]);
        }
        if (park_it && last) {
          // This warp's rows of the partial sums are written: publish them (one count per epilogue warp).
          __threadfence();
          __syncwarp();
          if (lane == 0) add_release_gpu(p.park_flags + w.park_slot, 1);
        }
      }
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ transform: P operand generator
    const int tt = threadIdx.x - 8 * 32;
    const int n = tt % BN;       // column of the tile owned by this thread
    constexpr int NG = Cfg::NGROUPS;
    const int grp = tt / BN;     // this thread's group takes k-blocks with i % NGROUPS == grp
    uint32_t it = 0, tcount = 0;
    bool ok = true;
    LtWork work(p, KBT);
    for (LtItem w; ok && work.next(w); ++tcount) {
      int r, n0, s0;
      decode(w.tile, r, n0, s0);
      const int kcol = n0 + n;
      const bool col_ok = kcol < p.K;
      const float* a_col = p.a + static_cast<int64_t>(r) * p.a_s0 + static_cast<int64_t>(kcol) * p.a_s2;
      const float* b_col = p.b + static_cast<int64_t>(r) * p.b_s0 + static_cast<int64_t>(kcol) * p.b_s2;

      // Column maxima over the full I and J, clamped as the reference does (baselines/lt2exp.py:15-19): an
      // all -inf column gets -1e38, its exps are exact zeros and the result is -inf, never NaN.  The transform
      // threads split the rows: with 16-byte loads a thread takes four adjacent columns and every RG-th row,
      // otherwise its own column and every NG-th row; partial maxima meet in shared memory.
      float* part = mpart + (tcount & 1) * Cfg::MPART;
      int nparts = 0;
      if (p.ma_in != nullptr) {
        // the caller knows the maxima (a previous layer's epilogue produced them): no scan
      } else if (p.vec_ab) {
        const int q = tt % Cfg::CQ, rg = tt / Cfg::CQ;
        float4 pa = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY), pb = pa;
        if (n0 + 4 * q < p.K) {  // K is a multiple of 4 here: the quad is inside or outside as a whole
          pa = quad_column_max(p.a + static_cast<int64_t>(r) * p.a_s0 + n0 + 4 * q, p.a_s1, p.I, rg, Cfg::RG);
          pb = quad_column_max(p.b + static_cast<int64_t>(r) * p.b_s0 + n0 + 4 * q, p.b_s1, p.J, rg, Cfg::RG);
        }
        *reinterpret_cast<float4*>(part + rg * BN + 4 * q) = pa;
        *reinterpret_cast<float4*>(part + (Cfg::RG + rg) * BN + 4 * q) = pb;
        nparts = Cfg::RG;
      } else {
        part[grp * BN + n] = col_ok ? strided_column_max(a_col, p.a_s1, p.I, grp, NG) : -INFINITY;
        part[(Cfg::RG + grp) * BN + n] = col_ok ? strided_column_max(b_col, p.b_s1, p.J, grp, NG) : -INFINITY;
        nparts = NG;
      }
      float ma = -INFINITY, mb = -INFINITY;
      if (p.ma_in != nullptr) {
        if (col_ok) {
          ma = __ldg(p.ma_in + static_cast<int64_t>(r) * p.K + kcol);
          mb = __ldg(p.mb_in + static_cast<int64_t>(r) * p.K + kcol);
        }
      } else {
        __syncwarp();
        if (lane == 0) mbar_arrive(mx_bar);
        if (!(ok = mbar_wait_warp(mx_bar, tcount & 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
        for (int g = 0; g < nparts; ++g) {
          ma = fmaxf(ma, part[g * BN + n]);
          mb = fmaxf(mb, part[(Cfg::RG + g) * BN + n]);
        }
      }
      ma = clamp_stab(ma);
      mb = clamp_stab(mb);
      const int slot = tcount & 1;
      if (grp == 0) {
        if (!(ok = mbar_wait_warp(&msum_empty[slot], ((tcount >> 1) & 1) ^ 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
        msum[slot * BN + n] = ma + mb;
      }

      for (int jc = w.kb_lo / p.I; ok && jc * p.I < w.kb_hi; ++jc) {
        const int i_lo = lt_row_lo(w, jc, p.I);
        const int In = lt_row_hi(w, jc, p.I) - i_lo;                             // rows of this j-chunk in the item
        const float* a_sl = a_col + static_cast<int64_t>(i_lo) * p.a_s1;  // the first of them
        // exp(b - mb) for this thread's column and the 32 j of the chunk; zero past J or K.
        // All 32 loads are issued before the first exp: padding reads as -inf, which exp turns into an exact
        // zero, so no exp sits behind a branch.
        float eb[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const int j = jc * BK + x;
          eb[x] = -INFINITY;
          if (col_ok && j < p.J) eb[x] = __ldg(b_col + static_cast<int64_t>(j) * p.b_s1);
        }
#pragma unroll
        for (int x = 0; x < 32; ++x) eb[x] = exp_shifted(eb[x], mb);
        // Raw a values of this group's next PF k-blocks.
        float apf[PF];
#pragma unroll
        for (int x = 0; x < PF; ++x) {
          const int i = grp + x * NG;  // row within the slice
          apf[x] = (col_ok && i < In) ? __ldg(a_sl + static_cast<int64_t>(i) * p.a_s1) : -INFINITY;
        }
        for (int ib = 0; ok && ib < In; ib += PF * NG) {
          float acur[PF];
#pragma unroll
          for (int x = 0; x < PF; ++x) {
            acur[x] = apf[x];
            const int i = ib + PF * NG + grp + x * NG;
            apf[x] = (col_ok && i < In) ? __ldg(a_sl + static_cast<int64_t>(i) * p.a_s1) : -INFINITY;
          }
#pragma unroll
          for (int x = 0; x < PF; ++x) {
            const int i = ib + grp + x * NG;
            if (i >= In) break;
            const uint32_t my_it = it + static_cast<uint32_t>(i);  // stage counter of k-block (jc, i_lo + i)
            const int s = my_it % NS;
            const uint32_t ph = (my_it / NS) & 1;
            if (!(ok = mbar_wait_warp(&opnd_empty[s], ph ^ 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
            const float ea = exp_shifted(acur[x], ma);  // acur = -inf past K: exact zero
            uint8_t* bh = b_tile(s, 0);
            uint8_t* bl = b_tile(s, PREC ? 1 : 0);
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const uint32_t off = static_cast<uint32_t>(n) * 128u + ((static_cast<uint32_t>(g) ^ (n & 7u)) << 4);
              const float p0 = ea * eb[g * 4 + 0], p1 = ea * eb[g * 4 + 1];
              const float p2 = ea * eb[g * 4 + 2], p3 = ea * eb[g * 4 + 3];
              if (PREC) {
                float4 h, l;
                tf32_split_rn(p0, h.x, l.x);
                tf32_split_rn(p1, h.y, l.y);
                tf32_split_rn(p2, h.z, l.z);
                tf32_split_rn(p3, h.w, l.w);
                *reinterpret_cast<float4*>(bh + off) = h;
                *reinterpret_cast<float4*>(bl + off) = l;
              } else {
                uint4 u;
                u.x = tf32_round_bits(p0);
                u.y = tf32_round_bits(p1);
                u.z = tf32_round_bits(p2);
                u.w = tf32_round_bits(p3);
                *reinterpret_cast<uint4*>(bh + off) = u;
              }
            }
            if (PREC) {
              // Split the w tiles in place (hi keeps the tf32 bits, lo = w - hi).
              if (!(ok = mbar_wait_warp(&a_full[s], ph, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
              float4* ah = reinterpret_cast<float4*>(a_tile(s, 0, 0));
              float4* al = reinterpret_cast<float4*>(a_tile(s, 1, 0));
              for (int c = n; c < MT * Cfg::A_TILE / 16; c += BN) {
                const float4 v = ah[c];
                float4 h, l;
                tf32_split_trunc(v.x, h.x, l.x);
                tf32_split_trunc(v.y, h.y, l.y);
                tf32_split_trunc(v.z, h.z, l.z);
                tf32_split_trunc(v.w, h.w, l.w);
                ah[c] = h;
                al[c] = l;
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&b_full[s]);
          }
        }
        it += static_cast<uint32_t>(In);
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// Zero-fills the (possibly strided) output before a split launch accumulates into it.
__global__ void lt2exp_zero_kernel(float* out, int64_t out_s0, int64_t out_s1, int R, int S, int K) {
  const int64_t total = static_cast<int64_t>(R) * S * K;
  for (int64_t x = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; x < total;
       x += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int k = static_cast<int>(x % K);
    const int64_t rs = x / K;
    out[(rs / S) * out_s0 + (rs % S) * out_s1 + k] = 0.0f;
  }
}

// Second pass of a split launch: out[r,s,k] = (ma[r,k] + mb[r,k]) + log(out[r,s,k]) in place, with the same
// clamped column maxima the main kernel used.  Block = 128 columns x 64 rows of out, 256 threads; the
// maxima are taken as in the main kernel (32 column quads x 8 row groups with 16-byte loads, or 128 columns x
// 2 row groups).  Grid = (K / 128, S / 64, R).
template <int PREC>
__global__ void __launch_bounds__(256) lt2exp_finish_kernel(const Lt2expParams p) {
  __shared__ float part[2][8][128];
  __shared__ float msum[128];
  const int k0 = blockIdx.x * 128;
  const int r = blockIdx.z;
  const int tid = threadIdx.x;
  int nparts = 0;
  if (p.ma_in != nullptr) {
    if (tid < 128 && k0 + tid < p.K) {
      part[0][0][tid] = __ldg(p.ma_in + static_cast<int64_t>(r) * p.K + k0 + tid);
      part[1][0][tid] = __ldg(p.mb_in + static_cast<int64_t>(r) * p.K + k0 + tid);
    } else if (tid < 128) {
      part[0][0][tid] = part[1][0][tid] = -INFINITY;
    }
    nparts = 1;
  } else if (p.vec_ab) {
    const int q = tid & 31, rg = tid >> 5;
    float4 pa = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY), pb = pa;
    if (k0 + 4 * q < p.K) {
      pa = quad_column_max(p.a + static_cast<int64_t>(r) * p.a_s0 + k0 + 4 * q, p.a_s1, p.I, rg, 8);
      pb = quad_column_max(p.b + static_cast<int64_t>(r) * p.b_s0 + k0 + 4 * q, p.b_s1, p.J, rg, 8);
    }
    *reinterpret_cast<float4*>(&part[0][rg][4 * q]) = pa;
    *reinterpret_cast<float4*>(&part[1][rg][4 * q]) = pb;
    nparts = 8;
  } else {
    const int n = tid & 127, g = tid >> 7;
    const bool col_ok = k0 + n < p.K;
    part[0][g][n] = col_ok ? strided_column_max(p.a + static_cast<int64_t>(r) * p.a_s0 + static_cast<int64_t>(k0 + n) * p.a_s2, p.a_s1, p.I, g, 2) : -INFINITY;
    part[1][g][n] = col_ok ? strided_column_max(p.b + static_cast<int64_t>(r) * p.b_s0 + static_cast<int64_t>(k0 + n) * p.b_s2, p.b_s1, p.J, g, 2) : -INFINITY;
    nparts = 2;
  }
  __syncthreads();
  if (tid < 128) {
    float ma = -INFINITY, mb = -INFINITY;
    for (int g = 0; g < nparts; ++g) {
      ma = fmaxf(ma, part[0][g][tid]);
      mb = fmaxf(mb, part[1][g][tid]);
    }
    msum[tid] = clamp_stab(ma) + clamp_stab(mb);
  }
  __syncthreads();
  const int n = tid & 127;
  if (k0 + n >= p.K) return;
  const float m = msum[n];
  const int s_end = min(p.S, (static_cast<int>(blockIdx.y) + 1) * 64);
  float cmx = -INFINITY;  // maximum of this thread's results: its column, every second row of the block
  for (int s = blockIdx.y * 64 + (tid >> 7); s < s_end; s += 2) {
    float* o = p.out + static_cast<int64_t>(r) * p.out_s0 + static_cast<int64_t>(s) * p.out_s1 + k0 + n;
    const float acc = *o;
    const float res = m + (PREC ? logf(acc) : lg2_approx(acc) * LN2_F);
    *o = res;
    cmx = fmaxf(cmx, res);
  }
  if (p.out_max != nullptr) red_max_f32(p.out_max + static_cast<int64_t>(r) * p.K + k0 + n, cmx);
}

}  // namespace tb200
