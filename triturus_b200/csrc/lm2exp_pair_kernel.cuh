// lm2exp on CTA pairs (tcgen05 cta_group::2).  Same arithmetic and operand layouts as lm2exp_kernel.cuh
// (replaces triturus/lm2exp.py:63-164), but two CTAs on neighbouring SMs share one 256 x 256 output tile:
// each CTA loads its own 128 rows of a and its own 128 columns of b, turns those columns into the
// tf32-rounded exp(b - m) operand in place, and one thread of the leader CTA issues pair MMAs (M = 256,
// N = 256, K = 8) that run on both tensor cores: each CTA accumulates its 128 rows x 256 columns in its
// own TMEM.
//
// Compared with a single CTA working on 256 x 256, a stage is 32 KB instead of 64 KB (six stages instead
// of three cover the TMA latency), one exp feeds 256 MACs, and the accumulator takes 256 TMEM columns, so it
// is double-buffered and the epilogue of a tile overlaps the main loop of the next.
//
// Roles per CTA: warp 0 TMA producer, warp 1 TMEM allocation (+ MMA issue in the leader), warps 4-7
// epilogue, warps 8-15 transform.  Cross-CTA signalling: the transform warps of both CTAs arrive on the
// leader's xf_done barrier; the leader's MMA thread commits each stage to the stage_empty barrier of both
// CTAs and each finished tile to both acc_full barriers; the epilogue warps of both CTAs arrive on the
// leader's acc_empty barrier.  No TMA multicast is used.  The stabiliser m comes from the pre-pass.
#pragma once

#include "lm2exp_kernel.cuh"

namespace tb200 {

template <int PREC_, int NS_>
struct Lm2expPairCfg {
  static constexpr int BM = 128;   // rows per CTA (256 per pair)
  static constexpr int BN = 256;   // columns per pair tile
  static constexpr int BNH = 128;  // columns whose operand this CTA builds
  static constexpr int BK = 32, NTW = 8;
  static constexpr int PREC = PREC_, NS = NS_;
  static constexpr int NCOPY = PREC ? 2 : 1;
  static constexpr int A_TILE = BM * BK * 4;  // 16 KB
  static constexpr int B_BOX = 32 * BK * 4;   // 4 KB
  static constexpr int NGRP = BNH / 32;
  static constexpr int B_TILE = NGRP * B_BOX;  // 16 KB
  static constexpr int STAGE = NCOPY * (A_TILE + B_TILE);
  static constexpr int RP = NTW / NGRP;
  static constexpr int ROWS_PER_WARP = BK / RP;
  static constexpr int ACC_COLS = BN;
  static constexpr int NBUF = 2;
  static constexpr int TMEM_COLS = 512;
  static constexpr int NTHREADS = (8 + NTW) * 32;
  static constexpr int NTT = NTW * 32;
  static constexpr int EPI_STAGE = 4 * 32 * 128;
  static constexpr int CMAX_BYTES = 2 * BN * 4;  // column maxima of the result, two tiles in flight
  static constexpr int NBAR = 3 * NS + 13;
  static constexpr int SMEM_BYTES = 1024 + NS * STAGE + EPI_STAGE + CMAX_BYTES + NBAR * 8 + 64;
  static_assert(SMEM_BYTES <= 232448, "shared memory capacity");
};

template <class Cfg>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg::NTHREADS, 1)
lm2exp_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_out, const Lm2expParams p) {
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BNH = Cfg::BNH, BK = Cfg::BK, NS = Cfg::NS;
  constexpr int PREC = Cfg::PREC, NTW = Cfg::NTW, NGRP = Cfg::NGRP;

  // A conditional launch: runs only if the launch before it left the word up (same value for every thread of
  // both CTAs, read before any barrier or allocation exists).
  if (p.only_if != nullptr) {
    pdl_wait();
    if (*p.only_if == 0) return;
    if (blockIdx.x == 0 && threadIdx.x == 0 && p.reset_flag != nullptr) *p.reset_flag = 0;  // all its readers are done
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint8_t* epi_stage = smem + NS * Cfg::STAGE;  // 4 warps x 4 KB staging boxes, 1024-byte aligned
  int* colbuf = reinterpret_cast<int*>(epi_stage + Cfg::EPI_STAGE);  // [2][BN] see flush_tile_colmax
  uint64_t* bars = reinterpret_cast<uint64_t*>(colbuf + 2 * BN);
  uint64_t* full = bars;                  // [NS] this CTA's TMA bytes landed
  uint64_t* xf_done = bars + NS;          // [NS] (leader's copy is used) transform warps of both CTAs done
  uint64_t* stage_empty = bars + 2 * NS;  // [NS] pair MMAs reading the stage retired (committed by the leader)
  uint64_t* acc_full = bars + 3 * NS;     // [2] accumulator buffer complete (committed by the leader)
  uint64_t* acc_empty = acc_full + 2;     // [2] (leader's copy is used) epilogues of both CTAs drained it
  uint64_t* cm_bar = acc_empty + 2;       // [1] this CTA's two fold warps folded their blocks of the tile
  uint64_t* box_ready = cm_bar + 1;       // [4] epilogue warp q filled its staging box
  uint64_t* box_free = box_ready + 4;     // [4] the fold warp has read epilogue warp q's staging box
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(box_free + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;
  const AbortCtl ctl{abort_flag, p.status};

  auto a_tile = [&](int s, int c) -> uint8_t* { return stage_base + s * Cfg::STAGE + c * Cfg::A_TILE; };
  auto b_tile = [&](int s, int c) -> uint8_t* {
    return stage_base + s * Cfg::STAGE + Cfg::NCOPY * Cfg::A_TILE + c * Cfg::B_TILE;
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&xf_done[s], 2 * NTW);
      mbar_init(&stage_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 8);
    }
    mbar_init(cm_bar, 2);
    for (int s = 0; s < 4; ++s) {
      mbar_init(&box_ready[s], 1);
      mbar_init(&box_free[s], 1);
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
  for (int c = threadIdx.x; c < 2 * BN; c += Cfg::NTHREADS) colbuf[c] = NEG_INF_BITS;
  // Both CTAs must have initialised their barriers before either one signals across.
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int KB = (p.J + BK - 1) / BK;
  const int npairs = gridDim.x >> 1;
  const int pair = blockIdx.x >> 1;

  // Pair tile id -> (batch r, first column, first row of the 256 x 256 tile); row tiles vary fastest.
  auto decode = [&](int tile, int& r, int& n0, int& i0) {
    const int tm = tile % p.tiles_m;
    const int rest = tile / p.tiles_m;
    const int tn = rest % p.tiles_n;
    r = rest / p.tiles_n;
    n0 = tn * BN;
    i0 = tm * (2 * BM);
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (this CTA's halves)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < p.num_tiles; tile += npairs) {
        int r, n0, i0;
        decode(tile, r, n0, i0);
        const int my_i0 = i0 + static_cast<int>(rank) * BM;
        const int my_n0 = n0 + static_cast<int>(rank) * BNH;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % NS;
          const uint32_t ph = (it / NS) & 1;
          if (!(ok = mbar_wait(&stage_empty[s], ph ^ 1, ctl, STATUS_TIMEOUT_PRODUCER))) break;
          mbar_arrive_expect_tx(&full[s], Cfg::A_TILE + Cfg::B_TILE);
          if (p.a_mn) {
#pragma unroll
            for (int g = 0; g < BM / 32; ++g)
              tma_load_3d(a_tile(s, 0) + g * 4096, &tmap_a, &full[s], my_i0 + g * 32, kb * BK, r);
          } else {
            tma_load_3d(a_tile(s, 0), &tmap_a, &full[s], kb * BK, my_i0, r);
          }
#pragma unroll
          for (int g = 0; g < NGRP; ++g)
            tma_load_3d(b_tile(s, 0) + g * Cfg::B_BOX, &tmap_b, &full[s], my_n0 + g * 32, kb * BK, r);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ pair MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      // M = 256 over the pair, B MN-major; A MN-major too when a is a transposed view (bit 15)
      const uint32_t idesc = umma_idesc_tf32(2 * BM, BN) | (1u << 16) | (p.a_mn ? (1u << 15) : 0u);
      const uint32_t a_step = p.a_mn ? 64u : 2u;  // encoded address step per 8 contraction values
      // This one thread feeds both tensor cores, so its per-k-block overhead is kept minimal: descriptors
      // of stage 0 are built once (stage s adds s * STAGE / 16 to the encoded address), one barrier wait
      // (the transform warps waited for the TMA bytes before they arrived), one multicast commit.
      constexpr uint32_t STAGE_ENC = Cfg::STAGE >> 4;
      const uint64_t da_hi0 = p.a_mn ? umma_desc_mn_sw128_base32(smem_u32(a_tile(0, 0)), 4096)
                                     : umma_desc_k_sw128(smem_u32(a_tile(0, 0)));
      const uint64_t da_lo0 = p.a_mn ? umma_desc_mn_sw128_base32(smem_u32(a_tile(0, PREC ? 1 : 0)), 4096)
                                     : umma_desc_k_sw128(smem_u32(a_tile(0, PREC ? 1 : 0)));
      const uint64_t db_hi0 = umma_desc_mn_sw128_base32(smem_u32(b_tile(0, 0)), Cfg::B_BOX);
      const uint64_t db_lo0 = umma_desc_mn_sw128_base32(smem_u32(b_tile(0, PREC ? 1 : 0)), Cfg::B_BOX);
      uint32_t s = 0, ph = 0, tcount = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < p.num_tiles; tile += npairs, ++tcount) {
        const int buf = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!(ok = mbar_wait(&acc_empty[buf], aph ^ 1, ctl, STATUS_TIMEOUT_MMA))) break;
        tc_fence_after_sync();
        const uint32_t d = tmem_base + buf * Cfg::ACC_COLS;
        for (int kb = 0; kb < KB; ++kb) {
          if (!(ok = mbar_wait(&xf_done[s], ph, ctl, STATUS_TIMEOUT_MMA))) break;
          tc_fence_after_sync();
          const uint64_t da_hi = da_hi0 + s * STAGE_ENC, db_hi = db_hi0 + s * STAGE_ENC;
          const uint64_t da_lo = da_lo0 + s * STAGE_ENC, db_lo = db_lo0 + s * STAGE_ENC;
#pragma unroll
          for (int ks = 0; ks < BK / 8; ++ks) {
            const uint32_t acc = (kb > 0 || ks > 0) ? 1u : 0u;
            if (PREC) {
              umma_tf32_ss_pair(d, da_hi + a_step * ks, db_lo + 64 * ks, idesc, acc);
              umma_tf32_ss_pair(d, da_lo + a_step * ks, db_hi + 64 * ks, idesc, 1u);
              umma_tf32_ss_pair(d, da_hi + a_step * ks, db_hi + 64 * ks, idesc, 1u);
            } else {
              umma_tf32_ss_pair(d, da_hi + a_step * ks, db_hi + 64 * ks, idesc, acc);
            }
          }
          // free the stage in both CTAs once these MMAs retire
          umma_commit_pair_mcast(smem_u32(&stage_empty[s]), 3);
          if (++s == NS) {
            s = 0;
            ph ^= 1;
          }
        }
        if (ok) umma_commit_pair_mcast(smem_u32(&acc_full[buf]), 3);
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------------ epilogue (this CTA's 128 rows x 256 columns)
    const int q = warp & 3;
    uint8_t* stg = epi_stage + q * 4096;
    const bool use_tma = p.out_tma != 0;
    pdl_wait();  // m comes from the pre-pass, which may still be running when this kernel starts
    uint32_t tcount = 0, nblk = 0;  // tiles seen; staging boxes handed to the fold warp so far
    bool ok = true;
    // Optimistic pre-pass (the stabilisers are the column maxima over the first 32 rows only): a result that
    // overflowed raises *opt_flag and the caller's conditional launches redo the call with the exact maxima.
    const bool opt = p.opt_flag != nullptr;
    bool overflowed = false;
    const bool emit_max = p.out_max != nullptr;
    for (int tile = pair; ok && tile < p.num_tiles; tile += npairs, ++tcount) {
      int r, n0, i0;
      decode(tile, r, n0, i0);
      const int buf = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      if (!(ok = mbar_wait_warp(&acc_full[buf], aph, ctl, STATUS_TIMEOUT_EPILOGUE))) break;
      tc_fence_after_sync();
      const uint32_t acc_empty_leader = map_to_cta(smem_u32(&acc_empty[buf]), 0);
      const int rbase = i0 + static_cast<int>(rank) * BM + q * 32;
      float* out_r = p.out + static_cast<int64_t>(r) * p.out_s0;
      const float* mrow = p.m_ws + static_cast<int64_t>(r) * p.K;
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * Cfg::ACC_COLS;
      const bool rows_exist = i0 + static_cast<int>(rank) * BM < p.I;
      const int nchunks = rows_exist ? min(BN / 32, (p.K - n0 + 31) / 32) : 0;
      if (nchunks == 0) {
        // nothing to store (this CTA's rows are padding): release the buffer right away
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
        continue;
      }
      uint32_t v[2][32];
      tmem_ld_32x32(tbase, v[0]);
#pragma unroll 1
      for (int idx = 0; ok && idx < nchunks; idx += 2) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int c = idx + h;
          if (c < nchunks) {
            const int k0 = n0 + c * 32;
            const float m_lane = (k0 + lane < p.K) ? clamp_stab(__ldg(mrow + k0 + lane)) : 0.f;
            tmem_ld_wait();  // chunk c is in v[h]
            if (c + 1 < nchunks) {
              tmem_ld_32x32(tbase + (c + 1) * 32, v[h ^ 1]);
            } else {
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
            }
            float o[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float m_e = __shfl_sync(0xffffffffu, m_lane, e);
              const float acc = __uint_as_float(v[h][e]);
              o[e] = m_e + (PREC ? logf(acc) : lg2_approx(acc) * LN2_F);
            }
            if (opt) {
#pragma unroll
              for (int e = 0; e < 32; ++e) overflowed |= !(o[e] < INFINITY);  // +inf or NaN
            }
            // swizzled 32 x 32 staging box, then TMA store or row-wise stores (see lm2exp_kernel.cuh)
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
              // the next layer's stabiliser: the box goes to this warp's fold warp (see lm2exp_kernel.cuh)
              __syncwarp();
              if (lane == 0) mbar_arrive(&box_ready[q]);
              ++nblk;
            }
          }
        }
      }
    }
    if (use_tma && lane == 0) tma_store_wait_all();
    if (opt && __any_sync(0xffffffffu, overflowed) && lane == 0) *p.opt_flag = 1;
  } else if (warp >= 2 && warp < 4 && p.out_max != nullptr) {
    // ------------------------------------------------------------------ fold: column maxima of the result
    // As in lm2exp_kernel.cuh: warp 2 serves epilogue warps 4 and 5, warp 3 serves 6 and 7.  The other CTA of
    // the pair and the other row tiles add their maxima with the same global reduction.
    const int fw = warp - 2;
    uint32_t nb[2] = {0, 0};
    uint32_t mcount = 0;  // tiles whose column maxima this CTA has written
    bool ok = true;
    for (int tile = pair; ok && tile < p.num_tiles; tile += npairs) {
      int r, n0, i0;
      decode(tile, r, n0, i0);
      const int my_i0 = i0 + static_cast<int>(rank) * BM;
      if (my_i0 >= p.I) continue;  // this CTA's rows are padding: its epilogue stages nothing
      const int slot = mcount & 1;
      const int nchunks = min(BN / 32, (p.K - n0 + 31) / 32);
      for (int c = 0; ok && c < nchunks; ++c) {
#pragma unroll
        for (int qq = 0; qq < 2; ++qq) {
          const int q = 2 * fw + qq;
          if (!(ok = mbar_wait_warp(&box_ready[q], nb[qq] & 1, ctl, STATUS_TIMEOUT_EPILOGUE))) break;
          ++nb[qq];
          fold_staged_colmax(epi_stage + q * 4096, p.I - (my_i0 + q * 32), colbuf + slot * BN + c * 32, lane,
                             &box_free[q]);
        }
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(cm_bar);
      if (!(ok = mbar_wait_warp(cm_bar, mcount & 1, ctl, STATUS_TIMEOUT_EPILOGUE))) break;
      flush_tile_colmax(colbuf + slot * BN, BN, p.out_max + static_cast<int64_t>(r) * p.K + n0, p.K - n0, false,
                        fw * 32 + lane);
      ++mcount;
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ transform: this CTA's b boxes -> E, in place
    const int wv = warp - 8;
    const int grp = wv % NGRP;
    const int rp = wv / NGRP;
    const int c = lane & 7;
    const int jsub = lane >> 3;
    const int tt = threadIdx.x - 8 * 32;
    uint32_t it = 0;
    bool ok = true;
    pdl_wait();  // m comes from the pre-pass (the producer warp is already loading operand tiles meanwhile)
    for (int tile = pair; ok && tile < p.num_tiles; tile += npairs) {
      int r, n0, i0;
      decode(tile, r, n0, i0);
      const int col0 = n0 + static_cast<int>(rank) * BNH + grp * 32 + c * 4;
      const float* mrow = p.m_ws + static_cast<int64_t>(r) * p.K;
      float m4[4];
      bool colv[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        colv[x] = col0 + x < p.K;
        m4[x] = colv[x] ? clamp_stab(__ldg(mrow + col0 + x)) : 0.f;
      }
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int s = it % NS;
        const uint32_t ph = (it / NS) & 1;
        if (!(ok = mbar_wait_warp(&full[s], ph, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
        uint8_t* box_hi = b_tile(s, 0) + grp * Cfg::B_BOX;
        uint8_t* box_lo = b_tile(s, PREC ? 1 : 0) + grp * Cfg::B_BOX;
        const int jrem = p.J - kb * BK;
        constexpr int NLD = Cfg::ROWS_PER_WARP / 4;
        // loads, then arithmetic, then stores (the stores overwrite what the loads read)
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
          // padding rows / columns: -inf in, exact zero out (the TMA zero fill is in log space)
          const bool rowv = j < jrem;
          float e[4];
          e[0] = exp_shifted((rowv && colv[0]) ? v[x].x : -INFINITY, m4[0]);
          e[1] = exp_shifted((rowv && colv[1]) ? v[x].y : -INFINITY, m4[1]);
          e[2] = exp_shifted((rowv && colv[2]) ? v[x].z : -INFINITY, m4[2]);
          e[3] = exp_shifted((rowv && colv[3]) ? v[x].w : -INFINITY, m4[3]);
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
        if (PREC) {
          float4* ah = reinterpret_cast<float4*>(a_tile(s, 0));
          float4* al = reinterpret_cast<float4*>(a_tile(s, 1));
          for (int ch = tt; ch < Cfg::A_TILE / 16; ch += Cfg::NTT) {
            const float4 w = ah[ch];
            float4 h, l;
            tf32_split_trunc(w.x, h.x, l.x);
            tf32_split_trunc(w.y, h.y, l.y);
            tf32_split_trunc(w.z, h.z, l.z);
            tf32_split_trunc(w.w, h.w, l.w);
            ah[ch] = h;
            al[ch] = l;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        // the MMA issuer lives in the leader CTA: both CTAs report there
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&xf_done[s]), 0));
      }
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
}

}  // namespace tb200
