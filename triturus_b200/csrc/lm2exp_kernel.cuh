// lm2exp:  out[r,i,k] = m[r,k] + log( sum_j a[r,i,j] * exp(b[r,j,k] - m[r,k]) ),  m = clamp(max_j b, +-1e38)
//
// Replaces the reference's Triton kernel _ker_lm2exp (triturus/lm2exp.py:63-164) with one persistent,
// warp-specialised sm_100a kernel.  As a GEMM: D[M = i, N = k] = A[M, Kc = j] * E[Kc, N], E = exp(b - m).
//
// b is N-major in memory (k contiguous), so E is used as an MN-major tensor-core operand: TMA drops each
// 32 j-rows x 32 k-columns box of b (128-byte rows, 128-byte swizzle with 32-byte base, the one swizzled
// layout tf32 MN-major operands may use) straight into the operand stage and the
// transform warps replace it IN PLACE by tf32-rounded exp(b - m): one 16-byte shared-memory load, four ex2,
// one 16-byte store per thread and step, no second buffer and no transposition.
//
//   warp 0      TMA producer: per k-block MT a-tiles (128 x 32 fp32, K-major, 128B swizzle) and BN/32 b-boxes.
//   warp 1      allocates TMEM; one lane issues tcgen05.mma.kind::tf32 (M = 128, N = BN, K = 8) and commits.
//   warps 2-3   only when the column maxima of the result are wanted (chain links): read the epilogue warps'
//               staged blocks back and fold them into max_i out[i, k], one value per tile column.
//   warps 4-7   epilogue: tcgen05.ld, out = m + log(acc), staged per warp as a swizzled 32 x 32 box in shared
//               memory and written by TMA stores (full 128-byte rows, clipped at the edges).
//   warps 8-15  transform.  Warp w owns the 32-column group w % (BN/32); lane = 8 * row_slot + 16-byte chunk.
//
// Stabiliser.  Either m comes from a pre-pass through the caller's workspace, or (fused_max) every tile
// starts with a max pass: the same b boxes stream through the ring once more, the transform warps keep a
// running maximum per column and fold the four row slots of a warp with shuffles.  The fused form reads b
// from HBM once and again from L2; it is chosen when each column slab of b is used by a single row tile.
//
// One CTA tile is (MT * 128) rows x BN columns; the MT row blocks share each generated operand.
// Accumulators live in TMEM (MT * BN columns per buffer, double-buffered when 2 * MT * BN <= 512).
// PREC = 1 selects the 3xTF32 split: a = a_hi + a_lo, e = e_hi + e_lo and
// acc += a_hi*e_lo + a_lo*e_hi + a_hi*e_hi.
#pragma once

#include "ptx.cuh"

namespace tb200 {

struct Lm2expParams {
  const float* m_ws;       // [R, K] column maxima of b (read only when fused_max == 0; clamped on read)
  float* out;              // [R, I, K]
  float* out_max;          // [R, K] receives max_i out[r,i,k], or nullptr; pre-filled with -inf by the
                           // caller unless a single row tile covers I (then every column is stored once)
  int64_t out_s0, out_s1;  // element strides of out (innermost stride is 1)
  int R, I, J, K;
  int tiles_m, tiles_n, num_tiles;
  int fused_max;
  int out_tma;              // out meets the TMA rules: the epilogue stores through tmap_out
  int a_mn;                 // a is stored with i contiguous (a transposed view): MN-major A operand, loaded as
                            // four 32 i x 32 j boxes per 128-row tile in the layout of the b boxes
  int b_km = 0;             // b is stored with j contiguous (a transposed view): K-major B operand, one 32 j x BN k
                            // box per stage in the 128-byte swizzle, exp'd in place row by row; pre-pass stabiliser only
  // Operands that break the tensor-map rules (a row pitch that is not a multiple of 16 bytes, an innermost stride
  // other than 1, an unaligned base) are fetched element by element with 4-byte asynchronous copies by warps 2-3
  // into the same swizzled stages; gen_a / gen_b say which, the pointers and element strides are theirs.
  int gen_a = 0, gen_b = 0;
  const float* a_ptr = nullptr;
  const float* b_ptr = nullptr;
  int64_t a_s0 = 0, a_s1 = 0, a_s2 = 0, b_s0 = 0, b_s1 = 0, b_s2 = 0;
  int* status;
  // The optimistic stabilisers (TMEM-operand pair kernel; fused max pass of the single-CTA kernel):
  const int* only_if = nullptr;  // a conditional launch: the kernel returns at once when *only_if == 0
  int* opt_flag = nullptr;       // optimistic launches set *opt_flag = 1 when a result overflowed
  int* reset_flag = nullptr;     // a conditional launch that does run puts this flag down: at once when only_if is a
                                 // republished copy of it (pair kernels), else by its last CTA, counted in reset_flag[1]
};

// PLAIN_ = true turns the kernel into a plain batched matrix product out = a * b (the reference's `mm`,
// triturus/mm.py:181-214): no stabiliser, no exp, no log; in the single-pass TF32 mode both operands are rounded
// to nearest tf32 as the reference's kernel does with cvt.rna (triturus/mm.py:152-154, triturus/utils.py:56-63).
// ODD_ = true adds the paths for operands in other layouts: a transposed b (p.b_km) and operands fetched element
// by element (p.gen_a / p.gen_b).  They are a template switch, not only run-time branches, because the kernel is
// sensitive to its code size: with those paths compiled into every instance the ordinary ones ran 5-14 % slower
// (cfg3 on the 128 x 2 tile with the full max pass 0.61 -> 0.70 ms, cfg1 at R = 64 20.6 -> 22.6 us).
template <int BN_, int MT_, int PREC_, int NS_, bool PROMOTE_ = (PREC_ != 0), bool PLAIN_ = false, bool ODD_ = false>
struct Lm2expCfg {
  static constexpr bool ODD = ODD_;
  static constexpr int BM = 128, BK = 32, NTW = 8;
  static constexpr int BN = BN_, MT = MT_, PREC = PREC_, NS = NS_;
  static constexpr bool PLAIN = PLAIN_;
  static constexpr int NCOPY = PREC ? 2 : 1;               // hi (+ lo) copies of each operand
  static constexpr int A_TILE = BM * BK * 4;               // 16 KB
  static constexpr int B_BOX = 32 * BK * 4;                // one 32-column group: 4 KB
  static constexpr int NGRP = BN / 32;
  static constexpr int B_TILE = NGRP * B_BOX;
  static constexpr int STAGE = NCOPY * (MT * A_TILE + B_TILE);
  static constexpr int RP = NTW / NGRP;                    // warps sharing one column group (row parts)
  static constexpr int ROWS_PER_WARP = BK / RP;
  static constexpr int ACC_COLS = MT * BN;
  static constexpr int NBUF = (2 * ACC_COLS <= 512) ? 2 : 1;
  // 3xTF32, and the plain-TF32 PROMOTE instances: contractions longer than CHUNK k-blocks are accumulated chunk by chunk and the chunks are
  // added into a master copy in TMEM with rounded fp32 adds (the tensor core's own accumulation truncates:
  // measured drift 2.6e-4 in log space at J = 16 K, 2.4e-3 at J = 256 K).  The master copy takes the TMEM
  // columns from MASTER_COL on; with 256 accumulator columns that is the second buffer, so a promoting
  // launch runs single-buffered.
  static constexpr bool PROMOTE = PROMOTE_;
  static constexpr int CHUNK = PREC ? 32 : 128;  // plain TF32 (PROMOTE instances, J > 32 K): every 4 K terms
  static constexpr int MASTER_COL = (ACC_COLS <= 128) ? 2 * ACC_COLS : ACC_COLS;
  static constexpr int NBUF_PROMOTE = (ACC_COLS <= 128) ? 2 : 1;
  static constexpr int TMEM_USED = PROMOTE ? (MASTER_COL + ACC_COLS) : NBUF * ACC_COLS;
  static constexpr int TMEM_COLS = (TMEM_USED <= 128) ? 128 : (TMEM_USED <= 256 ? 256 : 512);
  static_assert(!PROMOTE || ACC_COLS <= 256, "no room for the master copy");
  static constexpr int NTHREADS = (8 + NTW) * 32;
  static constexpr int NTT = NTW * 32;
  static constexpr int EPI_STAGE = 4 * 32 * 128;           // per epilogue warp one 32 x 32 fp32 box, 128B-swizzled
  static constexpr int MSUM_BYTES = 2 * BN * 4;
  static constexpr int MPART_BYTES = 2 * NTW * 32 * 4;
  static constexpr int CMAX_BYTES = 2 * BN * 4;            // column maxima of the result, two tiles in flight
  static constexpr int NBAR = 3 * NS + 16;
  static constexpr int SMEM_BYTES =
      1024 + NS * STAGE + EPI_STAGE + MSUM_BYTES + MPART_BYTES + CMAX_BYTES + NBAR * 8 + 64;
  static_assert(BN == 128 || BN == 256, "BN");
  static_assert(NTW % NGRP == 0 && ROWS_PER_WARP % 4 == 0, "transform warp mapping");
  static_assert(TMEM_USED <= 512, "TMEM capacity");
  static_assert(SMEM_BYTES <= 232448, "shared memory capacity");
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
lm2exp_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
              const __grid_constant__ CUtensorMap tmap_out, const Lm2expParams p) {
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, MT = Cfg::MT, NS = Cfg::NS;
  constexpr int PREC = Cfg::PREC, NTW = Cfg::NTW, NGRP = Cfg::NGRP, RP = Cfg::RP;
  // operands in other layouts (only instances built with ODD carry the code)
  const bool b_km = Cfg::ODD && p.b_km != 0;
  const bool gen_a = Cfg::ODD && p.gen_a != 0, gen_b = Cfg::ODD && p.gen_b != 0;

  // A conditional launch: runs only if the launch before it left the word up (same value for every thread,
  // read before any barrier or allocation exists).
  if (p.only_if != nullptr) {
    pdl_wait();
    if (*p.only_if == 0) return;
  }

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128B-swizzled tiles.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;                                          // NS stages of [A copies | B copies]
  uint8_t* epi_stage = smem + NS * Cfg::STAGE;                         // 4 warps x 4 KB, 1024-byte aligned
  float* msum = reinterpret_cast<float*>(epi_stage + Cfg::EPI_STAGE);  // [2][BN] stabiliser of the tile's columns
  float* mpart = msum + 2 * BN;                                        // [2][NTW][32] per-warp partial maxima
  int* colbuf = reinterpret_cast<int*>(mpart + 2 * NTW * 32);         // [2][BN] see flush_tile_colmax
  uint64_t* bars = reinterpret_cast<uint64_t*>(colbuf + 2 * BN);
  uint64_t* full = bars;                   // [NS] TMA bytes of the stage landed
  uint64_t* xf_done = bars + NS;           // [NS] transform warps finished with the stage
  uint64_t* stage_empty = bars + 2 * NS;   // [NS] stage may be overwritten
  uint64_t* acc_full = bars + 3 * NS;      // [2] accumulator buffer complete
  uint64_t* acc_empty = acc_full + 2;      // [2] epilogue drained the buffer
  uint64_t* msum_empty = acc_empty + 2;    // [2] epilogue finished reading msum[slot]
  uint64_t* mx_bar = msum_empty + 2;       // [1] all transform warps published their partial maxima
  uint64_t* cm_bar = mx_bar + 1;           // [1] both fold warps folded their blocks of the tile
  uint64_t* box_ready = cm_bar + 1;        // [4] epilogue warp q filled its staging box
  uint64_t* box_free = box_ready + 4;      // [4] the fold warp has read epilogue warp q's staging box
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(box_free + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AbortCtl ctl{abort_flag, p.status};

  // A tile copy c (0 = hi/raw, 1 = lo) of row block t in stage s; B copy c in stage s.
  auto a_tile = [&](int s, int c, int t) -> uint8_t* {
    return stage_base + s * Cfg::STAGE + (c * MT + t) * Cfg::A_TILE;
  };
  auto b_tile = [&](int s, int c) -> uint8_t* {
    return stage_base + s * Cfg::STAGE + Cfg::NCOPY * MT * Cfg::A_TILE + c * Cfg::B_TILE;
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], 1 + ((gen_a || gen_b) ? 64 : 0));  // + the 64 threads of the element-wise loader
      mbar_init(&xf_done[s], NTW);
      mbar_init(&stage_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 4);
      mbar_init(&msum_empty[s], 4);
    }
    mbar_init(mx_bar, NTW);
    mbar_init(cm_bar, 2);
    for (int s = 0; s < 4; ++s) {
      mbar_init(&box_ready[s], 1);
      mbar_init(&box_free[s], 1);
    }
    fence_mbar_init();
    if (!gen_a) tma_prefetch_desc(&tmap_a);  // (a tensor map that is not used is all zeros)
    if (!gen_b) tma_prefetch_desc(&tmap_b);
    if (p.out_tma) tma_prefetch_desc(&tmap_out);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  for (int c = threadIdx.x; c < 2 * BN; c += Cfg::NTHREADS) colbuf[c] = NEG_INF_BITS;
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int KB = (p.J + BK - 1) / BK;  // k-blocks per pass
  const bool fused = p.fused_max != 0;
  // Optimistic fused max pass: only the first k-block of a tile's slab is scanned for the stabiliser; values
  // further down may exceed it (exp(b - m) > 1, which fp32 holds up to e^88), and a result that overflowed all
  // the same raises *opt_flag, upon which the caller's conditional launch redoes the call with the full pass.
  const bool opt = fused && p.opt_flag != nullptr;
  const int KBM = opt ? 1 : KB;  // k-blocks of the max pass
  if (opt) {
    // the conditional launch behind this one may take its place as this grid's CTAs leave; the word behind the
    // flag, with which that launch finds its last CTA should it run, is cleared here (nothing else uses it now)
    pdl_launch_dependents();
    if (blockIdx.x == 0 && threadIdx.x == 0) p.opt_flag[1] = 0;
  }
  // Accumulation chunks per tile and the accumulator buffers they rotate through (see Lm2expCfg::PROMOTE).
  const bool promote = Cfg::PROMOTE && KB > Cfg::CHUNK;
  const int nch = promote ? (KB + Cfg::CHUNK - 1) / Cfg::CHUNK : 1;
  const int nbuf = promote ? Cfg::NBUF_PROMOTE : Cfg::NBUF;

  // Tile id -> (batch r, column tile, row tile); row tiles vary fastest so CTAs that run together
  // share one b slab in L2.
  auto decode = [&](int tile, int& r, int& n0, int& i0) {
    const int tm = tile % p.tiles_m;
    const int rest = tile / p.tiles_m;
    const int tn = rest % p.tiles_n;
    r = rest / p.tiles_n;
    n0 = tn * BN;
    i0 = tm * (BM * MT);
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        int r, n0, i0;
        decode(tile, r, n0, i0);
        // With the fused max pass the next tile's b slab is pulled into L2 while this tile computes, so
        // that its max pass (the first touch of that slab) streams from L2 instead of waiting on HBM
        // with only NS stages in flight.
        int nr = 0, nn0 = 0, ni0 = 0;
        const bool prefetch_next = fused && tile + static_cast<int>(gridDim.x) < p.num_tiles;
        if (prefetch_next) decode(tile + gridDim.x, nr, nn0, ni0);
        for (int pass = fused ? 0 : 1; ok && pass < 2; ++pass) {  // 0 = max pass (b only), 1 = contraction
          for (int kb = 0; kb < (pass ? KB : KBM); ++kb, ++it) {
            const int s = it % NS;
            const uint32_t ph = (it / NS) & 1;
            if (!(ok = mbar_wait(&stage_empty[s], ph ^ 1, ctl, STATUS_TIMEOUT_PRODUCER))) break;
            mbar_arrive_expect_tx(&full[s], ((pass && !gen_a) ? MT * Cfg::A_TILE : 0) + (gen_b ? 0 : Cfg::B_TILE));
            if (pass && !gen_a) {
              if (p.a_mn) {
#pragma unroll
                for (int t = 0; t < MT; ++t) {
#pragma unroll
                  for (int g = 0; g < BM / 32; ++g)
                    tma_load_3d(a_tile(s, 0, t) + g * 4096, &tmap_a, &full[s], i0 + t * BM + g * 32, kb * BK, r);
                }
              } else {
#pragma unroll
                for (int t = 0; t < MT; ++t) tma_load_3d(a_tile(s, 0, t), &tmap_a, &full[s], kb * BK, i0 + t * BM, r);
              }
            }
            if (pass && prefetch_next && !gen_b) {
#pragma unroll
              for (int g = 0; g < NGRP; ++g) tma_prefetch_l2_3d(&tmap_b, nn0 + g * 32, kb * BK, nr);
            }
            if (gen_b) {
              // (warps 2-3 fetch the b tile)
            } else if (b_km) {
              tma_load_3d(b_tile(s, 0), &tmap_b, &full[s], kb * BK, n0, r);  // rows k of 32 j: the layout of an a tile
            } else {
#pragma unroll
              for (int g = 0; g < NGRP; ++g)
                tma_load_3d(b_tile(s, 0) + g * Cfg::B_BOX, &tmap_b, &full[s], n0 + g * 32, kb * BK, r);
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // B operand is MN-major; A too when a is a transposed view (bit 15)
      const uint32_t idesc = umma_idesc_tf32(BM, BN) | (b_km ? 0u : (1u << 16)) | (p.a_mn ? (1u << 15) : 0u);
      const uint32_t a_step = p.a_mn ? 64u : 2u;  // encoded address step per 8 contraction values
      const uint32_t b_step = b_km ? 2u : 64u;  // K-major: 32 bytes along the row; MN-major: eight 128-byte rows
      uint32_t it = 0, ccount = 0;  // k-block stages and accumulation chunks issued so far
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        if (fused) {
          // Max-pass stages carry no MMA work: hand them back as soon as the transform warps are done.
          for (int kb = 0; kb < KBM; ++kb, ++it) {
            const int s = it % NS;
            const uint32_t ph = (it / NS) & 1;
            if (!(ok = mbar_wait(&xf_done[s], ph, ctl, STATUS_TIMEOUT_MMA))) break;
            mbar_arrive(&stage_empty[s]);
          }
          if (!ok) break;
        }
        int kb = 0;
        for (int ch = 0; ok && ch < nch; ++ch, ++ccount) {
          const int buf = ccount % nbuf;
          const uint32_t aph = (ccount / nbuf) & 1;
          if (!(ok = mbar_wait(&acc_empty[buf], aph ^ 1, ctl, STATUS_TIMEOUT_MMA))) break;
          tc_fence_after_sync();
          const int kb0 = kb;
          const int kb_end = promote ? min(KB, kb0 + Cfg::CHUNK) : KB;
          for (; kb < kb_end; ++kb, ++it) {
            const int s = it % NS;
            const uint32_t ph = (it / NS) & 1;
            if (!(ok = mbar_wait(&full[s], ph, ctl, STATUS_TIMEOUT_MMA))) break;
            if (!(ok = mbar_wait(&xf_done[s], ph, ctl, STATUS_TIMEOUT_MMA))) break;
            tc_fence_after_sync();
            const uint64_t db_hi = b_km ? umma_desc_k_sw128(smem_u32(b_tile(s, 0)))
                                          : umma_desc_mn_sw128_base32(smem_u32(b_tile(s, 0)), Cfg::B_BOX);
            const uint64_t db_lo = !PREC ? 0
                                   : b_km ? umma_desc_k_sw128(smem_u32(b_tile(s, 1)))
                                            : umma_desc_mn_sw128_base32(smem_u32(b_tile(s, 1)), Cfg::B_BOX);
#pragma unroll
            for (int t = 0; t < MT; ++t) {
              const uint32_t d = tmem_base + buf * Cfg::ACC_COLS + t * BN;
              const uint64_t da_hi = p.a_mn ? umma_desc_mn_sw128_base32(smem_u32(a_tile(s, 0, t)), 4096)
                                            : umma_desc_k_sw128(smem_u32(a_tile(s, 0, t)));
              const uint64_t da_lo = !PREC ? 0
                                     : p.a_mn ? umma_desc_mn_sw128_base32(smem_u32(a_tile(s, 1, t)), 4096)
                                              : umma_desc_k_sw128(smem_u32(a_tile(s, 1, t)));
#pragma unroll
              for (int ks = 0; ks < BK / 8; ++ks) {
                // One MMA consumes 8 contraction values: 32 bytes along a K-major row of A, eight
                // 128-byte rows (two 512-byte swizzle atoms) of the MN-major B boxes.
                const uint32_t acc = (kb > kb0 || ks > 0) ? 1u : 0u;
                if (PREC) {
                  umma_tf32_ss(d, da_hi + a_step * ks, db_lo + b_step * ks, idesc, acc);
                  umma_tf32_ss(d, da_lo + a_step * ks, db_hi + b_step * ks, idesc, 1u);
                  umma_tf32_ss(d, da_hi + a_step * ks, db_hi + b_step * ks, idesc, 1u);
                } else {
                  umma_tf32_ss(d, da_hi + a_step * ks, db_hi + b_step * ks, idesc, acc);
                }
              }
            }
            umma_commit(&stage_empty[s]);
          }
          if (ok) umma_commit(&acc_full[buf]);
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint8_t* stg = epi_stage + q * 4096;  // this warp's staging box
    const bool use_tma = p.out_tma != 0;
    uint32_t tcount = 0, ccount = 0;
    uint32_t nblk = 0;  // staging boxes handed to the fold warp so far
    bool ok = true;
    bool overflowed = false;  // optimistic max pass: some result of this lane came out +inf or NaN
    const bool emit_max = p.out_max != nullptr;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcount) {
      int r, n0, i0;
      decode(tile, r, n0, i0);
      const int slot = tcount & 1;
      // 32-column chunks of this tile that hold real rows / columns, in (row block, column chunk) order.
      const int nt = min(MT, (p.I - i0 + BM - 1) / BM);
      const int nc = min(BN / 32, (p.K - n0 + 31) / 32);
      const int nchunks = nt * nc;
      int buf = 0;
      for (int ch = 0; ok && ch < nch; ++ch, ++ccount) {
        buf = ccount % nbuf;
        const uint32_t aph = (ccount / nbuf) & 1;
        if (!(ok = mbar_wait_warp(&acc_full[buf], aph, ctl, STATUS_TIMEOUT_EPILOGUE))) break;
        tc_fence_after_sync();
        if (Cfg::PROMOTE && promote) {
          // Accumulation chunk `ch` of a long contraction: the first one becomes the master copy, the
          // following ones are added to it, and the last sum is written back over the chunk so that the
          // output code below finds the whole contraction in `buf`.
          const bool last = ch == nch - 1;
          const uint32_t part = lane_base + buf * Cfg::ACC_COLS;
          const uint32_t master = lane_base + Cfg::MASTER_COL;
#pragma unroll 1
          for (int cur = 0; cur < nchunks; ++cur) {
            const int t = cur / nc, c = cur - t * nc;
            uint32_t v[32];
            tmem_ld_32x32(part + t * BN + c * 32, v);
            if (ch > 0) {
              uint32_t mv[32];
              tmem_ld_32x32(master + t * BN + c * 32, mv);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 32; ++e)
                v[e] = __float_as_uint(__fadd_rn(__uint_as_float(v[e]), __uint_as_float(mv[e])));
            } else {
              tmem_ld_wait();
            }
            tmem_st_32x32((last ? part : master) + t * BN + c * 32, v);
          }
          tmem_st_wait();
          if (!last) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
          }
        }
      }
      if (!ok) break;
      float* out_r = p.out + static_cast<int64_t>(r) * p.out_s0;
      const uint32_t tbase = lane_base + buf * Cfg::ACC_COLS;
      // The TMEM load of the next chunk is in flight while one chunk is processed.
      uint32_t v[2][32];
      tmem_ld_32x32(tbase, v[0]);
#pragma unroll 1
      for (int idx = 0; ok && idx < nchunks; idx += 2) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int cur = idx + h;
          if (cur < nchunks) {
            const int t = cur / nc, c = cur - t * nc;
            tmem_ld_wait();  // chunk `cur` is in v[h]
            if (cur + 1 < nchunks) {
              const int t1 = (cur + 1) / nc, c1 = (cur + 1) - t1 * nc;
              tmem_ld_32x32(tbase + t1 * BN + c1 * 32, v[h ^ 1]);
            } else {
              // every accumulator value of this tile is in registers: hand the buffer back to the MMA warp
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&acc_empty[buf]);
            }
            const int rbase = i0 + t * BM + q * 32;
            const int k0 = n0 + c * 32;
            const float4* m4p = reinterpret_cast<const float4*>(msum + slot * BN + c * 32);
            float o[32];
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const float4 m4 = m4p[g];  // same address in every lane: broadcast
              const float a0 = __uint_as_float(v[h][g * 4 + 0]), a1 = __uint_as_float(v[h][g * 4 + 1]);
              const float a2 = __uint_as_float(v[h][g * 4 + 2]), a3 = __uint_as_float(v[h][g * 4 + 3]);
              if (Cfg::PLAIN) {
                o[g * 4 + 0] = a0;
                o[g * 4 + 1] = a1;
                o[g * 4 + 2] = a2;
                o[g * 4 + 3] = a3;
              } else {
                o[g * 4 + 0] = m4.x + (PREC ? logf(a0) : lg2_approx(a0) * LN2_F);
                o[g * 4 + 1] = m4.y + (PREC ? logf(a1) : lg2_approx(a1) * LN2_F);
                o[g * 4 + 2] = m4.z + (PREC ? logf(a2) : lg2_approx(a2) * LN2_F);
                o[g * 4 + 3] = m4.w + (PREC ? logf(a3) : lg2_approx(a3) * LN2_F);
              }
            }
            if (opt) {
#pragma unroll
              for (int x = 0; x < 32; ++x) overflowed |= !(o[x] < INFINITY);  // +inf or NaN
            }
            // Row `lane` of the 32 x 32 block goes to this warp's staging box in the 128-byte swizzle
            // (16-byte chunk g at position g ^ (row % 8): conflict-free).
            // the fold warp (column maxima of the result) has read the previous box
            if (emit_max && nblk > 0 &&
                !(ok = mbar_wait_warp(&box_free[q], (nblk - 1) & 1, ctl, STATUS_TIMEOUT_EPILOGUE)))
              break;
            if (use_tma) {
              if (lane == 0) tma_store_wait_read<0>();  // the previous box has been read out
              __syncwarp();
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                *reinterpret_cast<float4*>(stg + lane * 128 + ((g ^ (lane & 7)) << 4)) =
                    make_float4(o[g * 4], o[g * 4 + 1], o[g * 4 + 2], o[g * 4 + 3]);
              }
              // one lane hands the box to the TMA unit, which writes full rows and clips at the tensor's edges
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&tmap_out, stg, k0, rbase, r);
                tma_store_commit();
              }
            } else {
              // The result does not meet the TMA rules (K not a multiple of 4, unaligned base): the warp
              // writes the box row by row, 32 consecutive floats per store instruction.
              __syncwarp();
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                *reinterpret_cast<float4*>(stg + lane * 128 + ((g ^ (lane & 7)) << 4)) =
                    make_float4(o[g * 4], o[g * 4 + 1], o[g * 4 + 2], o[g * 4 + 3]);
              }
              __syncwarp();
              if (k0 + lane < p.K)
                store_staged_rows(stg, out_r + static_cast<int64_t>(rbase) * p.out_s1 + k0 + lane, p.out_s1,
                                  min(32, p.I - rbase), lane);
            }
            if (emit_max) {
              // The next layer's stabiliser: the box goes to this warp's fold warp, which takes the column
              // maxima of the block off this warp's critical path.
              __syncwarp();
              if (lane == 0) mbar_arrive(&box_ready[q]);
              ++nblk;
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&msum_empty[slot]);
    }
    if (use_tma && lane == 0) tma_store_wait_all();  // shared memory must outlive the last box
    if (opt && __any_sync(0xffffffffu, overflowed) && lane == 0) *p.opt_flag = 1;
  } else if (warp >= 2 && warp < 4 && (gen_a || gen_b)) {
    // ------------------------------------------------------------------ element-wise loader (never with out_max)
    // Walks the stages exactly as the TMA producer does and fills the tiles of the operands it is responsible
    // for.  A stage is reported `LAG` stages late: each thread waits for its own copies of that stage
    // (cp.async groups), makes them visible to the tensor core's proxy and arrives on the stage's barrier.
    constexpr int LAG = NS > 2 ? 2 : 1;
    const int lt = threadIdx.x - 64;  // 0..63
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
      int r, n0, i0;
      decode(tile, r, n0, i0);
      const float* ar = p.a_ptr + static_cast<int64_t>(r) * p.a_s0;
      const float* br = p.b_ptr + static_cast<int64_t>(r) * p.b_s0;
      for (int pass = fused ? 0 : 1; ok && pass < 2; ++pass) {
        for (int kb = 0; kb < (pass ? KB : KBM); ++kb, ++it) {
          const int s = it % NS;
          const uint32_t ph = (it / NS) & 1;
          if (!(ok = mbar_wait_warp(&stage_empty[s], ph ^ 1, ctl, STATUS_TIMEOUT_PRODUCER))) break;
          const int j0 = kb * BK;
          if (pass && gen_a) {
            // a tile: 128 x MT rows i of 32 values j, K-major, 128-byte swizzle; consecutive threads consecutive j
            for (int e = lt; e < MT * BM * BK; e += 64) {
              const int row = e >> 5, j = e & 31;
              const int t = row >> 7, rr = row & 127;
              const bool valid = i0 + row < p.I && j0 + j < p.J;
              const float* src = ar + static_cast<int64_t>(i0 + row) * p.a_s1 + static_cast<int64_t>(j0 + j) * p.a_s2;
              cp_async_f32(smem_u32(a_tile(s, 0, t)) + sw128_offset(rr, j), valid ? src : p.a_ptr, valid);
            }
          }
          if (gen_b) {
            // b tile: 32 rows j of BN values k in boxes of 32 columns; consecutive threads consecutive k
            for (int e = lt; e < BK * BN; e += 64) {
              const int j = e / BN, k = e % BN;
              const bool valid = j0 + j < p.J && n0 + k < p.K;
              const float* src = br + static_cast<int64_t>(j0 + j) * p.b_s1 + static_cast<int64_t>(n0 + k) * p.b_s2;
              const uint32_t dst = smem_u32(b_tile(s, 0)) + (k >> 5) * Cfg::B_BOX + sw128_base32_offset(j, (k & 31) >> 2) +
                                   (k & 3) * 4;
              cp_async_f32(dst, valid ? src : p.b_ptr, valid);
            }
          }
          cp_async_commit();
          if (it >= LAG) {
            cp_async_wait<LAG>();
            fence_proxy_async_smem();
            mbar_arrive(&full[(it - LAG) % NS]);
          }
        }
      }
    }
    // the last LAG stages
    cp_async_wait<0>();
    fence_proxy_async_smem();
    if (ok) {
      for (uint32_t d = (it < LAG ? it : LAG); d > 0; --d) mbar_arrive(&full[(it - d) % NS]);
    }
  } else if (warp >= 2 && warp < 4 && p.out_max != nullptr) {
    // ------------------------------------------------------------------ fold: column maxima of the result
    // Warp 2 serves epilogue warps 4 and 5, warp 3 serves 6 and 7: it reads each staged 32 x 32 block of
    // results, hands the box back as soon as it holds it in registers, and folds the column maxima into the
    // tile's buffer; at the end of a tile the two fold warps write one value per column to global memory.
    const int fw = warp - 2;
    uint32_t nb[2] = {0, 0};
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcount) {
      int r, n0, i0;
      decode(tile, r, n0, i0);
      const int slot = tcount & 1;
      const int nt = min(MT, (p.I - i0 + BM - 1) / BM);
      const int nc = min(BN / 32, (p.K - n0 + 31) / 32);
      for (int cur = 0; ok && cur < nt * nc; ++cur) {  // the epilogue's block order
        const int t = cur / nc, c = cur - t * nc;
#pragma unroll
        for (int qq = 0; qq < 2; ++qq) {
          const int q = 2 * fw + qq;
          if (!(ok = mbar_wait_warp(&box_ready[q], nb[qq] & 1, ctl, STATUS_TIMEOUT_EPILOGUE))) break;
          ++nb[qq];
          fold_staged_colmax(epi_stage + q * 4096, p.I - (i0 + t * BM + q * 32), colbuf + slot * BN + c * 32, lane,
                             &box_free[q]);
        }
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(cm_bar);
      if (!(ok = mbar_wait_warp(cm_bar, tcount & 1, ctl, STATUS_TIMEOUT_EPILOGUE))) break;
      flush_tile_colmax(colbuf + slot * BN, BN, p.out_max + static_cast<int64_t>(r) * p.K + n0, p.K - n0,
                        p.tiles_m == 1, fw * 32 + lane);
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ transform: b boxes -> E operand, in place
    const int wv = warp - 8;
    const int grp = wv % NGRP;   // 32-column group of the tile owned by this warp
    const int rp = wv / NGRP;    // which ROWS_PER_WARP rows of each k-block this warp handles
    const int c = lane & 7;      // logical 16-byte chunk (4 columns) within the group
    const int jsub = lane >> 3;  // row slot: 4 rows per step
    const int tt = threadIdx.x - 8 * 32;
    uint32_t it = 0, tcount = 0, max_passes = 0;
    bool ok = true;
    if (!fused) pdl_wait();  // m comes from the pre-pass, which may still be running when this kernel starts
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcount) {
      int r, n0, i0;
      decode(tile, r, n0, i0);
      const int col0 = n0 + grp * 32 + c * 4;  // first of this thread's 4 columns
      float m4[4];
      // K-major b: a thread owns CPT 16-byte pieces of one row k of the tile (consecutive lanes, consecutive rows).
      constexpr int TPR = Cfg::NTT / BN, CPT = 8 / TPR;
      const int krow = tt % BN, kpart = tt / BN;

      if (fused) {
        // ---- max pass: running maximum of this thread's 4 columns over its row slots
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        for (int kb = 0; kb < KBM; ++kb, ++it) {
          const int s = it % NS;
          const uint32_t ph = (it / NS) & 1;
          if (!(ok = mbar_wait_warp(&full[s], ph, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
          const uint8_t* box = b_tile(s, 0) + grp * Cfg::B_BOX;
          const int jrem = p.J - kb * BK;
          float4 v[Cfg::ROWS_PER_WARP / 4];
#pragma unroll
          for (int x = 0; x < Cfg::ROWS_PER_WARP / 4; ++x) {
            const int j = rp * Cfg::ROWS_PER_WARP + 4 * x + jsub;
            v[x] = *reinterpret_cast<const float4*>(box + sw128_base32_offset(j, c));
          }
#pragma unroll
          for (int x = 0; x < Cfg::ROWS_PER_WARP / 4; ++x) {
            const int j = rp * Cfg::ROWS_PER_WARP + 4 * x + jsub;
            if (j < jrem) {  // rows past J are zero-filled by TMA and must not enter the maximum
              mx[0] = fmaxf(mx[0], v[x].x);
              mx[1] = fmaxf(mx[1], v[x].y);
              mx[2] = fmaxf(mx[2], v[x].z);
              mx[3] = fmaxf(mx[3], v[x].w);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&xf_done[s]);
        }
        if (!ok) break;
        // fold the four row slots of the warp (lanes c, c+8, c+16, c+24 hold the same columns)
#pragma unroll
        for (int sh = 8; sh <= 16; sh <<= 1) {
#pragma unroll
          for (int x = 0; x < 4; ++x) mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], sh));
        }
        if (RP > 1) {
          // fold the RP warps that share this column group through shared memory (double-buffered by pass)
          float* part = mpart + (max_passes & 1) * NTW * 32;
          if (jsub == 0) *reinterpret_cast<float4*>(part + wv * 32 + c * 4) = make_float4(mx[0], mx[1], mx[2], mx[3]);
          __syncwarp();
          if (lane == 0) mbar_arrive(mx_bar);
          if (!(ok = mbar_wait_warp(mx_bar, max_passes & 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
#pragma unroll
          for (int o = 0; o < RP; ++o) {
            const float4 v = *reinterpret_cast<const float4*>(part + (o * NGRP + grp) * 32 + c * 4);
            mx[0] = fmaxf(mx[0], v.x);
            mx[1] = fmaxf(mx[1], v.y);
            mx[2] = fmaxf(mx[2], v.z);
            mx[3] = fmaxf(mx[3], v.w);
          }
        }
        ++max_passes;
#pragma unroll
        for (int x = 0; x < 4; ++x) m4[x] = clamp_stab(mx[x]);
      } else if (Cfg::PLAIN) {
#pragma unroll
        for (int x = 0; x < 4; ++x) m4[x] = 0.f;  // plain product: no stabiliser
      } else if (b_km) {
        m4[0] = (n0 + krow < p.K) ? clamp_stab(__ldg(p.m_ws + static_cast<int64_t>(r) * p.K + n0 + krow)) : 0.f;
        m4[1] = m4[2] = m4[3] = m4[0];
      } else {
        const float* mrow = p.m_ws + static_cast<int64_t>(r) * p.K;
#pragma unroll
        for (int x = 0; x < 4; ++x) m4[x] = (col0 + x < p.K) ? clamp_stab(__ldg(mrow + col0 + x)) : 0.f;
      }

      // publish the stabiliser of this tile's columns for the epilogue
      const int slot = tcount & 1;
      if (b_km) {
        if (kpart == 0) {  // (whole warps: BN is a multiple of 32)
          if (!(ok = mbar_wait_warp(&msum_empty[slot], ((tcount >> 1) & 1) ^ 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
          msum[slot * BN + krow] = m4[0];
        }
      } else if (rp == 0) {
        if (!(ok = mbar_wait_warp(&msum_empty[slot], ((tcount >> 1) & 1) ^ 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
        if (jsub == 0)
          *reinterpret_cast<float4*>(msum + slot * BN + grp * 32 + c * 4) = make_float4(m4[0], m4[1], m4[2], m4[3]);
      }
      bool colv[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) colv[x] = col0 + x < p.K;

      // ---- contraction pass: exp in place
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int s = it % NS;
        const uint32_t ph = (it / NS) & 1;
        if (!(ok = mbar_wait_warp(&full[s], ph, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
        uint8_t* box_hi = b_tile(s, 0) + grp * Cfg::B_BOX;
        uint8_t* box_lo = b_tile(s, PREC ? 1 : 0) + grp * Cfg::B_BOX;
        const int jrem = p.J - kb * BK;
        constexpr int NLD = Cfg::ROWS_PER_WARP / 4;
        if (b_km) {
          // Row krow of the tile is column n0 + krow of b with its 32 values j of this k-block: eight 16-byte
          // pieces, piece i at (i ^ (krow & 7)) * 16 of the 128-byte row.  Eight consecutive lanes read the same
          // piece index of eight consecutive rows, which the swizzle spreads over all 32 banks.
          uint8_t* rowp_hi = b_tile(s, 0) + krow * 128;
          uint8_t* rowp_lo = b_tile(s, PREC ? 1 : 0) + krow * 128;
          const bool kv = n0 + krow < p.K;
          float4 w[CPT];
#pragma unroll
          for (int x = 0; x < CPT; ++x)
            w[x] = *reinterpret_cast<const float4*>(rowp_hi + (((kpart * CPT + x) ^ (krow & 7)) << 4));
          uint4 whi[CPT];
          float4 wlo[CPT];
#pragma unroll
          for (int x = 0; x < CPT; ++x) {
            const int j0 = (kpart * CPT + x) * 4;
            float e[4];
            e[0] = exp_shifted((kv && j0 + 0 < jrem) ? w[x].x : -INFINITY, m4[0]);
            e[1] = exp_shifted((kv && j0 + 1 < jrem) ? w[x].y : -INFINITY, m4[0]);
            e[2] = exp_shifted((kv && j0 + 2 < jrem) ? w[x].z : -INFINITY, m4[0]);
            e[3] = exp_shifted((kv && j0 + 3 < jrem) ? w[x].w : -INFINITY, m4[0]);
            if (PREC) {
              float4 h;
              tf32_split_rn(e[0], h.x, wlo[x].x);
              tf32_split_rn(e[1], h.y, wlo[x].y);
              tf32_split_rn(e[2], h.z, wlo[x].z);
              tf32_split_rn(e[3], h.w, wlo[x].w);
              whi[x] = make_uint4(__float_as_uint(h.x), __float_as_uint(h.y), __float_as_uint(h.z), __float_as_uint(h.w));
            } else {
              whi[x] = make_uint4(tf32_round_bits(e[0]), tf32_round_bits(e[1]), tf32_round_bits(e[2]),
                                  tf32_round_bits(e[3]));
            }
          }
#pragma unroll
          for (int x = 0; x < CPT; ++x) {
            const uint32_t off = static_cast<uint32_t>(((kpart * CPT + x) ^ (krow & 7)) << 4);
            *reinterpret_cast<uint4*>(rowp_hi + off) = whi[x];
            if (PREC) *reinterpret_cast<float4*>(rowp_lo + off) = wlo[x];
          }
        } else {
        // All loads first, then the arithmetic, then all stores: the stores go to the addresses the loads
        // came from, so the compiler would otherwise serialise the iterations.
        float4 v[NLD];
#pragma unroll
        for (int x = 0; x < NLD; ++x) {
          const int j = rp * Cfg::ROWS_PER_WARP + 4 * x + jsub;
          v[x] = *reinterpret_cast<const float4*>(box_hi + sw128_base32_offset(j, c));
        }
        uint4 hi[NLD];
        float4 lo[NLD];
#pragma unroll
        for (int x = 0; x < NLD; ++x) {
          const int j = rp * Cfg::ROWS_PER_WARP + 4 * x + jsub;
          // Rows past J and columns past K must be exact zeros in the operand: the TMA zero fill is in
          // log space, and exp(0 - m) is not zero.
          // The mask is applied to the input (-inf gives an exact zero) so that the exps themselves
          // run unconditionally and interleave; a branch around each one would serialise them.
          const bool rowv = j < jrem;
          float e[4];
          if (Cfg::PLAIN) {
            // plain product: b itself is the operand (zeros in the padding)
            e[0] = (rowv && colv[0]) ? v[x].x : 0.f;
            e[1] = (rowv && colv[1]) ? v[x].y : 0.f;
            e[2] = (rowv && colv[2]) ? v[x].z : 0.f;
            e[3] = (rowv && colv[3]) ? v[x].w : 0.f;
          } else {
            e[0] = exp_shifted((rowv && colv[0]) ? v[x].x : -INFINITY, m4[0]);
            e[1] = exp_shifted((rowv && colv[1]) ? v[x].y : -INFINITY, m4[1]);
            e[2] = exp_shifted((rowv && colv[2]) ? v[x].z : -INFINITY, m4[2]);
            e[3] = exp_shifted((rowv && colv[3]) ? v[x].w : -INFINITY, m4[3]);
          }
          if (PREC) {
            float4 h;
            tf32_split_rn(e[0], h.x, lo[x].x);
            tf32_split_rn(e[1], h.y, lo[x].y);
            tf32_split_rn(e[2], h.z, lo[x].z);
            tf32_split_rn(e[3], h.w, lo[x].w);
            hi[x] = make_uint4(__float_as_uint(h.x), __float_as_uint(h.y), __float_as_uint(h.z), __float_as_uint(h.w));
          } else {
            hi[x] = make_uint4(tf32_round_bits(e[0]), tf32_round_bits(e[1]), tf32_round_bits(e[2]),
                               tf32_round_bits(e[3]));
          }
        }
#pragma unroll
        for (int x = 0; x < NLD; ++x) {
          const int j = rp * Cfg::ROWS_PER_WARP + 4 * x + jsub;
          const uint32_t off = sw128_base32_offset(j, c);
          *reinterpret_cast<uint4*>(box_hi + off) = hi[x];
          if (PREC) *reinterpret_cast<float4*>(box_lo + off) = lo[x];
        }
        }  // (MN-major b)
        if (PREC) {
          // Split the a-tiles in place: hi keeps the tf32 bits, lo = a - hi goes to the second copy.
          float4* ah = reinterpret_cast<float4*>(a_tile(s, 0, 0));
          float4* al = reinterpret_cast<float4*>(a_tile(s, 1, 0));
          for (int ch = tt; ch < MT * Cfg::A_TILE / 16; ch += Cfg::NTT) {
            const float4 v = ah[ch];
            float4 h, l;
            tf32_split_trunc(v.x, h.x, l.x);
            tf32_split_trunc(v.y, h.y, l.y);
            tf32_split_trunc(v.z, h.z, l.z);
            tf32_split_trunc(v.w, h.w, l.w);
            ah[ch] = h;
            al[ch] = l;
          }
        } else if (Cfg::PLAIN) {
          // Plain single-pass TF32 product: round a to the nearest tf32 as well (the tensor core would truncate).
          uint4* ah = reinterpret_cast<uint4*>(a_tile(s, 0, 0));
          for (int ch = tt; ch < MT * Cfg::A_TILE / 16; ch += Cfg::NTT) {
            uint4 v = ah[ch];
            v.x += 0x1000u;
            v.y += 0x1000u;
            v.z += 0x1000u;
            v.w += 0x1000u;
            ah[ch] = v;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&xf_done[s]);
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // Give copies and MMAs still in flight time to land before shared memory and TMEM are released.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if (p.reset_flag != nullptr && threadIdx.x == 0) {
    // A conditional launch that ran: every CTA read the flag when it started, so the CTA that finishes last puts
    // it down (the word behind it counts the finished CTAs).
    __threadfence();
    if (atomicAdd(p.reset_flag + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      p.reset_flag[1] = 0;
      p.reset_flag[0] = 0;
    }
  }
}

}  // namespace tb200
