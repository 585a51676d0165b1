// lt2exp with the generated operand in TENSOR MEMORY (TF32).
//
// Same contraction as lt2exp_kernel.cuh (which replaces triturus/lt2exp.py:227-357 and :365-506), computed
// transposed:
//
//     D^T[k, s] = sum_{(i,j)} P^T[k, (i,j)] * W^T[(i,j), s],   P^T[k, (i,j)] = exp(a[i,k]-ma[k]) * exp(b[j,k]-mb[k])
//
// so that the Khatri-Rao operand P^T is the tensor core's A operand, which tcgen05.mma can read from TMEM.  A
// transform thread owns one column k of the tile = one TMEM lane; per k-block (one i, 32 consecutive j) it
// forms its 32 products in registers and writes them to its lane with a single tcgen05.st.  The generated
// operand therefore never touches shared memory.  Per k-block the shared-memory pipe, which bounds
// lt2exp_kernel (w in, operand stores, operand reads), carries only the w tile: TMA in + one read by the
// tensor core (B operand, N = s, K-major as it lies in memory), which balances the tensor pipe exactly
// (128 x 256 x 32 MACs = 512 cycles; 64 KB at 128 B/clk = 512 cycles).
//
// Tile: 128 columns k (MMA M) x 128*MT rows s (MMA N, one instruction even for N = 256: the MT w boxes of a
// stage are contiguous and form one K-major tile).  The accumulator holds D^T: TMEM lane = k, column = s, so in
// the epilogue the 32 lanes of a warp hold 32 consecutive k of one output row, m = ma + mb is a per-lane
// constant and every store instruction writes one full 128-byte row segment.
//
// TMEM: NBUF accumulators of 128*MT columns (two when MT = 1) followed by NS operand stages of 32 columns.
// Stage s of shared memory (w) and operand stage s of TMEM are released together by one tcgen05.commit.
//
//   warp 0      TMA producer: w boxes {32 j, 1 i, 128 s, 1 r}, 128-byte swizzle.
//   warp 1      TMEM allocation; one lane issues tcgen05.mma.kind::tf32 with A in TMEM (M = 128, N = 128*MT, K = 8).
//   warps 4-7   epilogue: tcgen05.ld, out[s, k] = m[k] + log(acc), coalesced 128-byte stores (or fp32 reductions
//               into the zero-filled result when the contraction is split, see lt2exp_kernel.cuh).
//   warps 8-15  transform: warp w writes TMEM lane quarter w % 4; the two warps of a quarter take alternate
//               k-blocks.  Column maxima first (cooperative, as in lt2exp_kernel.cuh).
#pragma once

#include "lt2exp_kernel.cuh"

namespace tb200 {

template <int MT_, int NS_, int NB_ = 1>
struct Lt2expTmemCfg {
  static constexpr int BM = 128, BK = 32;  // BM: rows s per w box
  static constexpr int NB = NB_;           // 128-column blocks per tile: each is one M = 128 MMA on the same w tile
  static constexpr int BN = 128 * NB;      // columns k per tile
  static constexpr int MT = MT_, NS = NS_, PREC = 0, NTW = 8;
  static constexpr bool PROMOTE = false;  // no chunked re-summation of the accumulator in these kernels
  static constexpr int CHUNK = 1 << 30;
  static constexpr int W_TILE = BM * BK * 4;
  static constexpr int STAGE = MT * W_TILE;
  static constexpr int BLK_COLS = MT * BM;        // accumulator columns of one column block
  static constexpr int ACC_COLS = NB * BLK_COLS;
  static constexpr int P_STAGE = NB * BK;         // operand columns per stage
  static constexpr int NBUF = (2 * ACC_COLS + NS * P_STAGE <= 512) ? 2 : 1;
  static constexpr int P_COL0 = NBUF * ACC_COLS;  // first operand column
  static constexpr int TMEM_USED = P_COL0 + NS * P_STAGE;
  static constexpr int TMEM_COLS = 512;
  static constexpr int NTHREADS = (8 + NTW) * 32;
  static constexpr int NTT = NTW * 32;
  static constexpr int NGROUPS = NTT / BN;
  static constexpr int CQ = BN / 4;
  static constexpr int RG = NTT / CQ;
  static constexpr int MPART = 2 * RG * BN;
  static constexpr int NBAR = 3 * NS + 7;
  static constexpr int SMEM_BYTES = 1024 + NS * STAGE + 2 * BN * 4 + 2 * MPART * 4 + NBAR * 8 + 64;
  static_assert(TMEM_USED <= 512, "TMEM capacity");
  static_assert(NGROUPS * NB == 2, "eight transform warps: two groups on one column block, or one group on two");
  static_assert(SMEM_BYTES <= 232448, "shared memory capacity");
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
lt2exp_tmem_kernel(const __grid_constant__ CUtensorMap tmap_w, const Lt2expParams p) {
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, MT = Cfg::MT, NS = Cfg::NS;
  constexpr int PF = 8;  // prefetch distance (own k-blocks) for the a values

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  float* msum = reinterpret_cast<float*>(smem + NS * Cfg::STAGE);  // [2][BN]: ma + mb of the tile's columns
  float* mpart = msum + 2 * BN;                                    // [2][2][RG][BN] partial column maxima
  uint64_t* bars = reinterpret_cast<uint64_t*>(mpart + 2 * Cfg::MPART);
  uint64_t* full = bars;                 // [NS] w tile landed (TMA bytes) and operand stage written to TMEM
  uint64_t* opnd_empty = bars + 2 * NS;  // [NS] MMAs reading the stage (shared memory and TMEM) retired
  uint64_t* acc_full = bars + 3 * NS;    // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint64_t* msum_empty = acc_empty + 2;  // [2]
  uint64_t* mx_bar = msum_empty + 2;     // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mx_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AbortCtl ctl{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], 1 + Cfg::NTW / Cfg::NGROUPS);  // the producer and the warps that write the operand stage
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

  const int JC = (p.J + BK - 1) / BK;
  const int KBT = JC * p.I;  // k-blocks per output tile
  const bool split_mode = p.nsplit > 1 || p.stream != 0;

  // Output tile -> (r, n0 = first column k, s0 = first row s); the items of a CTA come from LtWork.
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
            mbar_arrive_expect_tx(&full[s], Cfg::STAGE);
#pragma unroll
            for (int t = 0; t < MT; ++t)
              tma_load_4d(stage_base + s * Cfg::STAGE + t * Cfg::W_TILE, &tmap_w, &full[s], jc * BK, i, s0 + t * BM, r);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop with uniform control flow and one elected lane issues, so stage indices,
    // descriptors and TMEM addresses stay in uniform registers.  One barrier per stage, and the barrier of
    // the next stage is polled before this stage's MMAs are issued so that the answer arrives meanwhile: a
    // single thread issuing four MMAs per k-block after two fresh barrier round trips took ~790 cycles per
    // k-block against 512 cycles of tensor work.
    {
      constexpr uint32_t idesc = umma_idesc_tf32(128, BM * MT);  // M = 128 columns k, N = rows s
      const uint32_t stage0 = smem_u32(stage_base);
      uint32_t tcount = 0;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true, ready = false;
      LtWork work(p, KBT);
      for (LtItem w; ok && work.next(w); ++tcount) {
        const int KB = w.kb_hi - w.kb_lo;
        const int buf = tcount % Cfg::NBUF;
        const uint32_t aph = (tcount / Cfg::NBUF) & 1;
        if (!(ok = mbar_wait_warp(&acc_empty[buf], aph ^ 1, ctl, STATUS_TIMEOUT_MMA))) break;
        tc_fence_after_sync();
        const uint32_t d = tmem_base + buf * Cfg::ACC_COLS;
        for (int kb = 0; kb < KB; ++kb) {
          if (!ready) {
            if (!(ok = mbar_wait_warp(&full[s], ph, ctl, STATUS_TIMEOUT_MMA))) break;
          }
          const int sn = (s + 1 == NS) ? 0 : s + 1;
          const uint32_t phn = (s + 1 == NS) ? ph ^ 1 : ph;
          const bool peek = mbar_try_wait(&full[sn], phn);
          tc_fence_after_sync();
          if (elect_one_sync()) {
            const uint64_t dw = umma_desc_k_sw128(stage0 + s * Cfg::STAGE);
            const uint32_t pa = tmem_base + Cfg::P_COL0 + s * Cfg::P_STAGE;
#pragma unroll
            for (int blk = 0; blk < Cfg::NB; ++blk) {  // the column blocks share the w tile
#pragma unroll
              for (int ks = 0; ks < BK / 8; ++ks)
                umma_tf32_ts(d + blk * Cfg::BLK_COLS, pa + blk * BK + ks * 8, dw + 2 * ks, idesc,
                             (kb > 0 || ks > 0) ? 1u : 0u);
            }
            umma_commit(&opnd_empty[s]);
          }
          ready = __all_sync(0xffffffffu, peek);
          s = sn;
          ph = phn;
        }
        if (ok && elect_one_sync()) umma_commit(&acc_full[buf]);
        __syncwarp();
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    uint32_t tcount = 0;
    bool ok = true;
    LtWork work(p, KBT);
    for (LtItem w; ok && work.next(w); ++tcount) {
      int r, n0, s0;
      decode(w.tile, r, n0, s0);
      const int buf = tcount % Cfg::NBUF;
      const uint32_t aph = (tcount / Cfg::NBUF) & 1;
      const int slot = tcount & 1;
      if (!(ok = mbar_wait_warp(&acc_full[buf], aph, ctl, STATUS_TIMEOUT_EPILOGUE))) break;
      tc_fence_after_sync();
#pragma unroll 1
      for (int blk = 0; blk < Cfg::NB; ++blk) {  // column blocks of the tile: this lane's column in each
        const int kcol = n0 + blk * 128 + q * 32 + lane;
        const bool col_ok = kcol < p.K;
        float* out_col = p.out + static_cast<int64_t>(r) * p.out_s0 + kcol;
        const float m = msum[slot * BN + blk * 128 + q * 32 + lane];
        float cmx = -INFINITY;  // running maximum of this lane's column over the rows of the tile
        // One chunk = 32 rows s for this lane's column.  The loop stays rolled (two chunks per trip, the
        // next one loading while the current one is finished): unrolled, every chunk was straight-line code
        // run once per tile and the epilogue ran at instruction-fetch speed (2 000-10 000 cycles per chunk).
        auto finish = [&](const uint32_t(&cur)[32], int sb) {
          if (split_mode) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              if (col_ok && sb + e < p.S)
                atomicAdd(out_col + static_cast<int64_t>(sb + e) * p.out_s1, __uint_as_float(cur[e]));
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float o = m + lg2_approx(__uint_as_float(cur[e])) * LN2_F;
              if (col_ok && sb + e < p.S) {
                out_col[static_cast<int64_t>(sb + e) * p.out_s1] = o;
                cmx = fmaxf(cmx, o);
              }
            }
          }
        };
        const uint32_t acc0 = lane_base + buf * Cfg::ACC_COLS + blk * Cfg::BLK_COLS;
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(acc0, v0);
#pragma unroll 1
        for (int c = 0; c < Cfg::BLK_COLS / 32; c += 2) {
          const int sb = s0 + c * 32;
          if (sb >= p.S) break;
          tmem_ld_wait();
          tmem_ld_32x32(acc0 + (c + 1) * 32, v1);
          finish(v0, sb);
          tmem_ld_wait();
          if (c + 2 < Cfg::BLK_COLS / 32) tmem_ld_32x32(acc0 + (c + 2) * 32, v0);
          if (sb + 32 < p.S) finish(v1, sb + 32);
        }
        tmem_ld_wait();
        if (p.out_max != nullptr && !split_mode && col_ok) {
          // the next layer's stabiliser: this lane owns the column, so the maximum is a register
          float* dst = p.out_max + static_cast<int64_t>(r) * p.K + kcol;
          if (p.tiles_m == 1) *dst = cmx;
          else red_max_f32(dst, cmx);
        }
      }
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&acc_empty[buf]);
        mbar_arrive(&msum_empty[slot]);
      }
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ transform: operand generator
    const int tt = threadIdx.x - 8 * 32;
    const int n = tt % BN;   // column of the tile = TMEM lane owned by this thread
    const int grp = tt / BN; // this thread's group takes k-blocks with (i - i_lo) % 2 == grp
    constexpr int NG = Cfg::NGROUPS;
    // TMEM lane quarter of this warp; with two column blocks per tile the upper four warps write the second
    // block's operand columns.
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + Cfg::P_COL0 +
                               (Cfg::NB == 2 ? static_cast<uint32_t>((tt / 128) * BK) : 0u);
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

      // Column maxima over the full I and J (see lt2exp_kernel.cuh).
      float* part = mpart + (tcount & 1) * Cfg::MPART;
      int nparts = 0;
      if (p.ma_in != nullptr) {
        // maxima supplied by the caller: no scan
      } else if (p.vec_ab) {
        const int q4 = tt % Cfg::CQ, rg = tt / Cfg::CQ;
        float4 pa = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY), pb = pa;
        if (n0 + 4 * q4 < p.K) {
          pa = quad_column_max(p.a + static_cast<int64_t>(r) * p.a_s0 + n0 + 4 * q4, p.a_s1, p.I, rg, Cfg::RG);
          pb = quad_column_max(p.b + static_cast<int64_t>(r) * p.b_s0 + n0 + 4 * q4, p.b_s1, p.J, rg, Cfg::RG);
        }
        *reinterpret_cast<float4*>(part + rg * BN + 4 * q4) = pa;
        *reinterpret_cast<float4*>(part + (Cfg::RG + rg) * BN + 4 * q4) = pb;
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
        const int In = lt_row_hi(w, jc, p.I) - i_lo;  // rows of this j-chunk in the item
        const float* a_sl = a_col + static_cast<int64_t>(i_lo) * p.a_s1;
        // exp(b - mb) of the 32 j of the chunk; padding (past J or K) enters the exp as -inf: exact zero.
        float eb[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const int j = jc * BK + x;
          eb[x] = -INFINITY;
          if (col_ok && j < p.J) eb[x] = __ldg(b_col + static_cast<int64_t>(j) * p.b_s1);
        }
#pragma unroll
        for (int x = 0; x < 32; ++x) eb[x] = exp_shifted(eb[x], mb);
        float apf[PF];
#pragma unroll
        for (int x = 0; x < PF; ++x) {
          const int i = grp + x * NG;
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
            const uint32_t my_it = it + static_cast<uint32_t>(i);
            const int s = my_it % NS;
            const uint32_t ph = (my_it / NS) & 1;
            const float ea = exp_shifted(acur[x], ma);
            uint32_t pv[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) pv[e] = tf32_round_bits(ea * eb[e]);
            if (!(ok = mbar_wait_warp(&opnd_empty[s], ph ^ 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
            tc_fence_after_sync();
            tmem_st_32x32(lane_base + s * Cfg::P_STAGE, pv);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
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

}  // namespace tb200
