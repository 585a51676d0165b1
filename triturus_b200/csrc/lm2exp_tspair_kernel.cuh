// lm2exp on CTA pairs with the generated operand in tensor memory (plain TF32).
//
// Same arithmetic as lm2exp_pair_kernel.cuh (replaces triturus/lm2exp.py:63-164), but the contraction is
// written transposed, D^T[k, i] = sum_j E^T[k, j] * a[i, j] with E = exp(b - m): the generated operand E^T is the
// tensor core's A operand, which tcgen05.mma can read from tensor memory, and `a` in its natural layout
// (j contiguous) is the K-major B operand.  A transform thread owns one column k of b = one TMEM lane: it
// reads its 32 values of a k-block from the b tile in shared memory (row j at 512-byte pitch, the 32 lanes of
// a warp read 128 consecutive bytes), takes the exps and writes them with one tcgen05.st.  The generated
// operand therefore never goes back to shared memory and is never read from it by the tensor core.
//
// Shared-memory bytes per k-block and CTA: 32 KB TMA in (128 rows of a, 128 columns of b), 16 KB transform
// reads, 16 KB tensor-core reads of a, 8 KB of result staging = 72 KB, against 124 KB for the kernel that keeps
// E in shared memory (which is bound by exactly that pipe: 970 cycles per k-block for 512 cycles of MMAs).
//
// One pair tile is 256 columns k (M, 128 per CTA = the CTA's TMEM lanes) x 256 rows i (N, 128 per CTA's
// shared memory).  Tensor memory per CTA: columns [0, 256) accumulator D^T, [256, 256 + 32 * NS) the E^T stages.
// The accumulator is single-buffered (a second one would leave no room for the operand), so the epilogue of a
// tile is not hidden behind the next tile's MMAs; the transform warps run ahead by NS k-blocks meanwhile.
// In the transposed result a lane owns a column k, so the stabiliser m[k] is a lane constant; a 32 x 32 block of
// results is staged in shared memory (the 32 lanes of a store fill one row) and written by one TMA store; two boxes per warp alternate.
//
//   warp 0      TMA producer of ring 1: this CTA's 128 rows of a (128B swizzle).
//   warp 1      TMEM allocation; in the leader CTA one lane issues the pair MMAs.
//   warp 2      TMA producer of ring 2: this CTA's 128 columns of b (no swizzle).
//   warp 3      watches the a tiles land and says so on the leader's xf_done barriers.
//   warps 4-7   epilogue (TMEM lane quarter = warp % 4).
//   warps 8-15  transform: NG = two groups of four warps (one per lane quarter) take alternate k-blocks (three
//               groups, 20 warps at 96 registers, ran 5 % slower; ring depths 6+6, 5+7, 7+5 instead of 8+4 the same).
#pragma once

#include "lm2exp_kernel.cuh"

namespace tb200 {

// Development aid (compiled only with -DTB200_TIMELINE, never in the shipped library): CTA 0 records clock64()
// at the hand-over points of its roles, 256 entries per slot.
#ifdef TB200_TIMELINE
__device__ long long g_timeline[16 * 256];
#define TB200_TL(slot, idx)                                                                  \
  do {                                                                                       \
    if (blockIdx.x == 0 && (idx) < 256u) g_timeline[(slot) * 256 + (idx)] = clock64();        \
  } while (0)
#else
#define TB200_TL(slot, idx) \
  do {                      \
  } while (0)
#endif

// Two rings.  Ring 1 (NS stages): a tile of `a` in shared memory together with the E^T stage in tensor memory
// that the same MMAs read; both are handed back by the MMA commit.  Ring 2 (NSB stages): the b tiles, which the
// transform threads hand back as soon as they hold the values in registers.  The chain "stage free -> TMA
// (1-2 us from L2 / HBM) -> transform -> MMA -> commit" is several thousand cycles long, so the number of
// k-blocks in flight, not any pipe, bounds a single ring of six stages (measured 1 100 cycles per k-block for
// 512 cycles of MMAs); two rings put 8 + 5 tiles in flight in the same shared memory.
template <int NS_, int NSB_, int NG_ = 2, bool OPT_ = false, bool FUSED_ = false>
struct Lm2expTsPairCfg {
  static constexpr int BM = 128;   // columns k per CTA (256 per pair): TMEM lanes
  static constexpr int BN = 256;   // rows i per pair tile (N of the MMA), 128 per CTA's shared memory
  static constexpr int BK = 32, NG = NG_, NTW = 4 * NG_, NS = NS_, NSB = NSB_;
  static constexpr int A_TILE = 128 * BK * 4;  // this CTA's rows of a: 16 KB
  static constexpr int B_TILE = BK * BM * 4;   // this CTA's columns of b: 32 rows j x 128 k = 16 KB
  static constexpr int ACC_COLS = BN;
  static constexpr int E_COL0 = ACC_COLS;  // first TMEM column of the operand stages
  static constexpr int TMEM_COLS = 512;
  static constexpr int NTHREADS = (8 + NTW) * 32;
  static constexpr int EPI_STAGE = 4 * 2 * 32 * 128;  // per epilogue warp two 32 x 32 fp32 boxes
  // OPT: no stabiliser pre-pass.  The stabiliser of a column is the maximum over its first k-block (32 rows j),
  // found by the transform warp that handles that k-block and handed to the other roles through shared memory
  // (two slots of 128 floats, per-quarter barriers).  Later values may exceed it: exp(b - m) then exceeds 1,
  // which fp32 absorbs up to e^88; a result that overflowed all the same (+inf or NaN) raises *opt_flag and the
  // caller's conditional launches redo the call with the exact column maxima.
  static constexpr bool OPT = OPT_;
  // FUSED: the exact stabiliser inside the kernel (the conditional launch behind an optimistic one).  Every tile
  // starts with a max pass: its b tiles stream through ring 2 once more, each transform group keeps the running
  // maximum of its k-blocks per lane, the groups other than the first hand theirs over through shared memory,
  // and the first group publishes the column maxima like the optimistic instance publishes its estimate.
  static constexpr bool FUSED = FUSED_;
  static constexpr bool SLOTS = OPT || FUSED;  // stabilisers handed from the transform warps to the other roles
  static_assert(!(OPT && FUSED), "one or the other");
  static constexpr int NBAR = 3 * NS + 2 * NSB + 2 + (SLOTS ? 16 : 0) + (FUSED ? 4 * (NG - 1) : 0);
  static constexpr int M_TILE_BYTES = (SLOTS ? 2 * BM * 4 : 0) + (FUSED ? (NG - 1) * BM * 4 : 0);
  static constexpr int SMEM_BYTES = 1024 + NS * A_TILE + NSB * B_TILE + EPI_STAGE + M_TILE_BYTES + NBAR * 8 + 64;
  static_assert(E_COL0 + NS * BK <= TMEM_COLS, "TMEM capacity");
  static_assert(SMEM_BYTES <= 232448, "shared memory capacity");
};

// D[tmem] (+)= A[tmem] * B[smem] on a CTA pair: each CTA supplies its 128 rows of A from its own tensor memory
// (same address in both) and its half of the N rows of B from its own shared memory (same offset in both).
__device__ __forceinline__ void umma_tf32_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], [%1], %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <class Cfg>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg::NTHREADS, 1)
lm2exp_tspair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_out, const Lm2expParams p) {
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, NS = Cfg::NS, NSB = Cfg::NSB;

  // A conditional launch: runs only if the launch before it raised the flag (same value for every thread of
  // both CTAs, read before any barrier or allocation exists).
  if (p.only_if != nullptr) {
    pdl_wait();  // (launched as a programmatic dependent of the kernel that may have raised the flag)
    if (*p.only_if == 0) return;
    // (a flag republished in a second word by a conditional pre-pass: all readers of the first one are done)
    if (!Cfg::FUSED && blockIdx.x == 0 && threadIdx.x == 0 && p.reset_flag != nullptr) *p.reset_flag = 0;
  }
  // Optimistic instances let the conditional launch behind them take its place as this grid's CTAs leave, and
  // clear the counter with which that launch, should it run, finds its last CTA (nothing else uses the word
  // while this kernel runs).
  if (Cfg::OPT) {
    pdl_launch_dependents();
    if (blockIdx.x == 0 && threadIdx.x == 0) p.opt_flag[1] = 0;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_base = smem;                     // ring 1: NS tiles of a
  uint8_t* b_base = smem + NS * Cfg::A_TILE;  // ring 2: NSB tiles of b
  uint8_t* epi_stage = b_base + NSB * Cfg::B_TILE;  // 4 warps x 4 KB staging boxes, 1024-byte aligned
  float* m_tile = reinterpret_cast<float*>(epi_stage + Cfg::EPI_STAGE);  // OPT: [2][BM] stabilisers of two tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + Cfg::EPI_STAGE + Cfg::M_TILE_BYTES);
  uint64_t* a_full = bars;                // [NS] this CTA's tile of a landed
  uint64_t* xf_done = bars + NS;          // [NS] (leader's copy is used) E^T stage written and a landed, both CTAs
  uint64_t* stage_empty = bars + 2 * NS;  // [NS] pair MMAs reading ring-1 stage retired (committed by the leader)
  uint64_t* b_full = bars + 3 * NS;       // [NSB] this CTA's tile of b landed
  uint64_t* b_empty = b_full + NSB;       // [NSB] the four transform warps of the k-block hold it in registers
  uint64_t* acc_full = b_empty + NSB;     // [1] accumulator complete (committed by the leader)
  uint64_t* acc_empty = acc_full + 1;     // [1] (leader's copy is used) epilogues of both CTAs drained it
  uint64_t* m_ready = acc_empty + 1;      // SLOTS [2][4] slot, lane quarter: stabilisers written
  uint64_t* m_free = m_ready + 8;         // SLOTS [2][4] every reader of the quarter (epilogue warp, other groups) is done
  uint64_t* part_ready = m_free + 8;      // FUSED [NG - 1][4] group g > 0, lane quarter: its partial maxima written
  float* m_part = m_tile + 2 * BM;        // FUSED [NG - 1][BM] partial column maxima of the groups other than the first
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1 + (Cfg::SLOTS ? 16 : 0) +
                                                    (Cfg::FUSED ? 4 * (Cfg::NG - 1) : 0));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;
  const AbortCtl ctl{abort_flag, p.status};

  auto a_tile = [&](int s) -> uint8_t* { return a_base + s * Cfg::A_TILE; };
  auto b_tile = [&](int s) -> uint8_t* { return b_base + s * Cfg::B_TILE; };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < NS; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&xf_done[s], 2 * 4 + 2);  // four transform warps (one per lane quarter) and the a-tile watcher, in each CTA
      mbar_init(&stage_empty[s], 1);
    }
    for (int s = 0; s < NSB; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&b_empty[s], 4);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 8);
    if (Cfg::SLOTS) {
      for (int i = 0; i < 8; ++i) {
        mbar_init(&m_ready[i], 1);
        mbar_init(&m_free[i], Cfg::NG);  // the epilogue warp and one warp of every other transform group
      }
    }
    if (Cfg::FUSED) {
      for (int i = 0; i < 4 * (Cfg::NG - 1); ++i) mbar_init(&part_ready[i], 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.out_tma) tma_prefetch_desc(&tmap_out);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  // Both CTAs must have initialised their barriers before either one signals across.
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int KB = (p.J + BK - 1) / BK;
  const int npairs = gridDim.x >> 1;
  const int pair = blockIdx.x >> 1;

  // Pair tile id -> (batch r, first column k, first row i of the 256 x 256 tile); row tiles vary fastest.
  auto decode = [&](int tile, int& r, int& n0, int& i0) {
    const int tm = tile % p.tiles_m;
    const int rest = tile / p.tiles_m;
    const int tn = rest % p.tiles_n;
    r = rest / p.tiles_n;
    n0 = tn * (2 * BM);
    i0 = tm * BN;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer, ring 1: this CTA's rows of a
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < p.num_tiles; tile += npairs) {
        int r, n0, i0;
        decode(tile, r, n0, i0);
        const int my_i0 = i0 + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % NS;
          const uint32_t ph = (it / NS) & 1;
          if (!(ok = mbar_wait(&stage_empty[s], ph ^ 1, ctl, STATUS_TIMEOUT_PRODUCER))) break;
          TB200_TL(9, it);
          mbar_arrive_expect_tx(&a_full[s], Cfg::A_TILE);
          tma_load_3d(a_tile(s), &tmap_a, &a_full[s], kb * BK, my_i0, r);
        }
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------------ TMA producer, ring 2: this CTA's columns of b
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < p.num_tiles; tile += npairs) {
        int r, n0, i0;
        decode(tile, r, n0, i0);
        const int my_n0 = n0 + static_cast<int>(rank) * BM;
        for (int pass = Cfg::FUSED ? 0 : 1; ok && pass < 2; ++pass) {  // 0 = max pass, 1 = contraction
          for (int kb = 0; kb < KB; ++kb, ++it) {
            const int s = it % NSB;
            const uint32_t ph = (it / NSB) & 1;
            if (!(ok = mbar_wait(&b_empty[s], ph ^ 1, ctl, STATUS_TIMEOUT_PRODUCER))) break;
            TB200_TL(10, it);
            mbar_arrive_expect_tx(&b_full[s], Cfg::B_TILE);
            tma_load_3d(b_tile(s), &tmap_b, &b_full[s], my_n0, kb * BK, r);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ pair MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      // M = 256 columns k over the pair (A from TMEM), N = 256 rows i (B = a, K-major, 128 rows per CTA)
      constexpr uint32_t idesc = umma_idesc_tf32(2 * BM, BN);
      constexpr uint32_t STAGE_ENC = Cfg::A_TILE >> 4;
      const uint64_t db0 = umma_desc_k_sw128(smem_u32(a_tile(0)));
      const uint32_t d = tmem_base;
      uint32_t s = 0, ph = 0, tcount = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < p.num_tiles; tile += npairs, ++tcount) {
        TB200_TL(11, tcount);
        if (!(ok = mbar_wait(acc_empty, (tcount & 1) ^ 1, ctl, STATUS_TIMEOUT_MMA))) break;
        TB200_TL(12, tcount);
        tc_fence_after_sync();
        for (int kb = 0; kb < KB; ++kb) {
          if (!(ok = mbar_wait(&xf_done[s], ph, ctl, STATUS_TIMEOUT_MMA))) break;
          TB200_TL(0, tcount * KB + kb);
          tc_fence_after_sync();
          const uint64_t db = db0 + s * STAGE_ENC;
          const uint32_t ea = tmem_base + Cfg::E_COL0 + s * BK;
#pragma unroll
          for (int ks = 0; ks < BK / 8; ++ks)
            umma_tf32_ts_pair(d, ea + ks * 8, db + 2 * ks, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
          // free the stage (shared memory and TMEM) in both CTAs once these MMAs retire
          umma_commit_pair_mcast(smem_u32(&stage_empty[s]), 3);
          TB200_TL(1, tcount * KB + kb);
          if (++s == NS) {
            s = 0;
            ph ^= 1;
          }
        }
        if (ok) umma_commit_pair_mcast(smem_u32(acc_full), 3);
      }
    }
    __syncwarp();
  } else if (warp == 3) {
    // ------------------------------------------------------------------ a-tile watcher
    // The leader's MMA thread reads both CTAs' tiles of a and waits only on xf_done: this lane adds "this CTA's
    // tile of a has landed" to that barrier, so that the transform warps need not wait for it in their chain.
    if (lane == 0) {
      const uint32_t xf_done_leader0 = map_to_cta(smem_u32(&xf_done[0]), 0);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < p.num_tiles; tile += npairs) {
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % NS;
          if (!(ok = mbar_wait(&a_full[s], (it / NS) & 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
          mbar_arrive_cluster(xf_done_leader0 + static_cast<uint32_t>(s) * 8u);
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------------ epilogue (this CTA's 128 columns k x 256 rows i)
    const int q = warp & 3;
    uint8_t* stg2 = epi_stage + q * 8192;  // two boxes: one is filled while the TMA unit still reads the other
    uint32_t nbox = 0;
    const bool use_tma = p.out_tma != 0;
    const uint32_t acc_empty_leader = map_to_cta(smem_u32(acc_empty), 0);
    const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    pdl_wait();  // m comes from the pre-pass, which may still be running when this kernel starts
    uint32_t tcount = 0;
    bool ok = true;
    uint32_t acc_max = 0;  // OPT: largest accumulator bit pattern of this lane (sums of non-negative products, so
                           // +inf and NaN are exactly the patterns >= 0x7f800000 read as unsigned)
    for (int tile = pair; ok && tile < p.num_tiles; tile += npairs, ++tcount) {
      int r, n0, i0;
      decode(tile, r, n0, i0);
      const int k0 = n0 + static_cast<int>(rank) * BM + q * 32;  // first column of this warp's 32
      const int kcol = k0 + lane;
      const bool col_ok = kcol < p.K;
      float m = 0.f;
      if (!Cfg::SLOTS && col_ok) m = clamp_stab(__ldg(p.m_ws + static_cast<int64_t>(r) * p.K + kcol));
      float* ocol = p.out + static_cast<int64_t>(r) * p.out_s0 + kcol;
      if (!(ok = mbar_wait_warp(acc_full, tcount & 1, ctl, STATUS_TIMEOUT_EPILOGUE))) break;
      if (warp == 4 && lane == 0) TB200_TL(7, tcount);
      tc_fence_after_sync();
      if (Cfg::SLOTS) {
        // the stabilisers this tile was computed with (written long before the accumulator completed)
        const uint32_t slot = (tcount & 1) * 4 + q;
        if (!(ok = mbar_wait_warp(&m_ready[slot], (tcount >> 1) & 1, ctl, STATUS_TIMEOUT_EPILOGUE))) break;
        const float mt = m_tile[(tcount & 1) * BM + q * 32 + lane];
        m = col_ok ? mt : 0.f;
        __syncwarp();
        if (lane == 0) mbar_arrive(&m_free[slot]);
      }
      const int nchunks = (k0 < p.K) ? min(BN / 32, (p.I - i0 + 31) / 32) : 0;
      if (nchunks == 0) {
        // nothing to store (this warp's columns are padding): release the accumulator right away
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
        continue;
      }
      uint32_t v[2][32];
      tmem_ld_32x32(tbase, v[0]);
#pragma unroll 1
      for (int idx = 0; idx < nchunks; idx += 2) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int c = idx + h;
          if (c < nchunks) {
            tmem_ld_wait();  // chunk c is in v[h]
            if (c + 1 < nchunks) {
              tmem_ld_32x32(tbase + (c + 1) * 32, v[h ^ 1]);
            } else {
              // the whole accumulator is in registers: hand it back to the MMA issuer
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
            }
            const int ib = i0 + c * 32;
            // Register e of this lane is row ib + e, column kcol of the result.  The 32 x 32 block goes through a
            // staging box (row e at byte e * 128 in the 128-byte swizzle, the 32 lanes of a store fill one row)
            // and from there as one TMA store: per-row stores straight from the registers ran at ~70 cycles per
            // row.
            if (use_tma) {
              uint8_t* stg = stg2 + (nbox & 1) * 4096;
              ++nbox;
              if (lane == 0) tma_store_wait_read<1>();  // the store before the previous one has read this box out
              __syncwarp();
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const float o = m + lg2_approx(__uint_as_float(v[h][e])) * LN2_F;
                if (Cfg::OPT) acc_max = max(acc_max, v[h][e]);
                *reinterpret_cast<float*>(stg + sw128_offset(e, lane)) = o;
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&tmap_out, stg, k0, ib, r);  // clipped at the edges of the tensor
                tma_store_commit();
              }
            } else {
              // A result that a TMA store cannot write (K not a multiple of 4, unaligned base): row by row.
              float* orow = ocol + static_cast<int64_t>(ib) * p.out_s1;
              const int nrows = min(32, p.I - ib);
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const float o = m + lg2_approx(__uint_as_float(v[h][e])) * LN2_F;
                if (Cfg::OPT) acc_max = max(acc_max, v[h][e]);
                if (col_ok && e < nrows) orow[static_cast<int64_t>(e) * p.out_s1] = o;
              }
            }
          }
        }
      }
      if (warp == 4 && lane == 0) TB200_TL(8, tcount);
    }
    if (use_tma && lane == 0) tma_store_wait_all();  // shared memory must outlive the last box
    if (Cfg::OPT) {
      if (__any_sync(0xffffffffu, acc_max >= 0x7f800000u) && lane == 0) *p.opt_flag = 1;
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ transform: b tile -> E^T in tensor memory
    const int q = warp & 3;         // TMEM lane quarter this warp may write
    const int grp = (warp - 8) >> 2;  // this warp's group takes the k-blocks with kb % NG == grp
    const int kl = q * 32 + lane;
    const uint32_t ebase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + Cfg::E_COL0;
    const uint32_t xf_done_leader0 = map_to_cta(smem_u32(&xf_done[0]), 0);
    pdl_wait();  // m comes from the pre-pass (the producer warp is already loading operand tiles meanwhile)
    uint32_t it0 = 0, itb0 = 0, tcount = 0;  // k-blocks of ring 1 / tiles of ring 2 before this tile; tiles seen
    bool ok = true;
    for (int tile = pair; ok && tile < p.num_tiles; tile += npairs, ++tcount) {
      int r, n0, i0;
      decode(tile, r, n0, i0);
      const int kcol = n0 + static_cast<int>(rank) * BM + kl;
      // A column past K reads zero-filled values; the stabiliser +inf turns them into exact zeros.
      float m = INFINITY;
      if (!Cfg::SLOTS && kcol < p.K) m = clamp_stab(__ldg(p.m_ws + static_cast<int64_t>(r) * p.K + kcol));
      const uint32_t mslot = (tcount & 1) * 4 + q;
      float* mdst = m_tile + (tcount & 1) * BM + kl;
      if (Cfg::FUSED) {
        // ---- max pass: running maximum of this lane's column over the k-blocks of this group
        float mx = -INFINITY;
        for (int kb = grp; kb < KB; kb += Cfg::NG) {
          const uint32_t itb = itb0 + static_cast<uint32_t>(kb);
          const int sb = itb % NSB;
          if (!(ok = mbar_wait_warp(&b_full[sb], (itb / NSB) & 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
          const float* col = reinterpret_cast<const float*>(b_tile(sb)) + kl;
          const int jrem = p.J - kb * BK;  // rows past J are zero-filled by TMA and must not enter the maximum
#pragma unroll
          for (int x = 0; x < 32; ++x) mx = fmaxf(mx, x < jrem ? col[x * BM] : -INFINITY);
          __syncwarp();
          if (lane == 0) mbar_arrive(&b_empty[sb]);
        }
        if (!ok) break;
        itb0 += static_cast<uint32_t>(KB);
        if (grp != 0) {
          // (rewritten only after this warp has seen m_ready of the tile, i.e. after the first group read it)
          m_part[(grp - 1) * BM + kl] = mx;
          __syncwarp();
          if (lane == 0) mbar_arrive(&part_ready[(grp - 1) * 4 + q]);
        } else {
          for (int g = 1; g < Cfg::NG; ++g) {
            if (!(ok = mbar_wait_warp(&part_ready[(g - 1) * 4 + q], tcount & 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
            mx = fmaxf(mx, m_part[(g - 1) * BM + kl]);
          }
          if (!ok) break;
          m = (kcol < p.K) ? clamp_stab(mx) : INFINITY;
          if (tcount >= 2) {
            if (!(ok = mbar_wait_warp(&m_free[mslot], ((tcount >> 1) - 1) & 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
          }
          *mdst = m;
          __syncwarp();
          if (lane == 0) mbar_arrive(&m_ready[mslot]);
        }
      }
      // The group of k-block 0 publishes the tile's stabilisers; the other groups pick them up.  In the optimistic
      // instance that is done after the loads of the group's own first k-block are in flight (the first group
      // publishes as soon as it holds k-block 0, i.e. at about the same time), not before them.
      bool need_m = Cfg::SLOTS && grp != 0;
      auto fetch_m = [&]() -> bool {
        if (!mbar_wait_warp(&m_ready[mslot], (tcount >> 1) & 1, ctl, STATUS_TIMEOUT_TRANSFORM)) return false;
        m = *mdst;
        __syncwarp();
        if (lane == 0) mbar_arrive(&m_free[mslot]);
        need_m = false;
        return true;
      };
      if (need_m && Cfg::FUSED) {
        if (!(ok = fetch_m())) break;
      }
      for (int kb = grp; kb < KB; kb += Cfg::NG) {
        const uint32_t it = it0 + static_cast<uint32_t>(kb);
        const int s = it % NS;
        const uint32_t ph = (it / NS) & 1;
        const uint32_t itb = itb0 + static_cast<uint32_t>(kb);
        const int sb = itb % NSB;
        if (!(ok = mbar_wait_warp(&b_full[sb], (itb / NSB) & 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
        if (warp == 8 && lane == 0) TB200_TL(2, it);
        const float* col = reinterpret_cast<const float*>(b_tile(sb)) + kl;
        float v[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) v[x] = col[x * BM];
        const int jrem = p.J - kb * BK;
        if (need_m) {
          if (!(ok = fetch_m())) break;
        }
        if (Cfg::OPT && kb == 0) {
          // (grp == 0) stabiliser = maximum over the first k-block; the slot's readers of two tiles ago are done
          float mx = -INFINITY;
#pragma unroll
          for (int x = 0; x < 32; ++x) mx = fmaxf(mx, x < jrem ? v[x] : -INFINITY);
          m = (kcol < p.K) ? clamp_stab(mx) : INFINITY;
          if (tcount >= 2) {
            if (!(ok = mbar_wait_warp(&m_free[mslot], ((tcount >> 1) - 1) & 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
          }
          *mdst = m;
          __syncwarp();
          if (lane == 0) mbar_arrive(&m_ready[mslot]);
        }
        uint32_t e[32];
        if (jrem >= BK) {
#pragma unroll
          for (int x = 0; x < 32; ++x) e[x] = tf32_round_bits(exp_shifted(v[x], m));
        } else {
          // rows past J are zero-filled by TMA (in log space): they enter the exp as -inf, exact zero out
#pragma unroll
          for (int x = 0; x < 32; ++x) e[x] = tf32_round_bits(exp_shifted(x < jrem ? v[x] : -INFINITY, m));
        }
        // Every lane has consumed its values of the b tile: hand the tile back to its producer.
        __syncwarp();
        if (lane == 0) mbar_arrive(&b_empty[sb]);
        // The E^T stage is free once the MMAs that read it last time have retired.  (That the tile of a the same
        // MMAs will read has landed is the watcher warp's part of xf_done.)
        if (!(ok = mbar_wait_warp(&stage_empty[s], ph ^ 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
        if (warp == 8 && lane == 0) TB200_TL(4, it);
        tc_fence_after_sync();
        tmem_st_32x32(ebase + s * BK, e);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(xf_done_leader0 + static_cast<uint32_t>(s) * 8u);
        if (warp == 8 && lane == 0) TB200_TL(6, it);
      }
      if (need_m) {  // (a group without a k-block in this tile still reads and releases the slot)
        if (!(ok = fetch_m())) break;
      }
      it0 += static_cast<uint32_t>(KB);
      itb0 += static_cast<uint32_t>(KB);
    }
  }

  // ------------------------------------------------------------------ teardown
  // Neither CTA may leave while the other can still signal into its shared memory or use its TMEM half.
  tc_fence_before_sync();
  cluster_sync_all();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
  if (Cfg::FUSED && p.reset_flag != nullptr && threadIdx.x == 0) {
    // A conditional launch that ran: every CTA read the flag when it started, so the CTA that finishes last may
    // put it down (the word behind it counts the finished CTAs; the optimistic launch before this one cleared it).
    __threadfence();
    if (atomicAdd(p.reset_flag + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      p.reset_flag[1] = 0;
      p.reset_flag[0] = 0;
    }
  }
}

}  // namespace tb200
