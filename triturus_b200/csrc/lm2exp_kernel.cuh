// lm2exp:  out[r,i,k] = m[r,k] + log( sum_j a[r,i,j] * exp(b[r,j,k] - m[r,k]) ),  m = clamp(max_j b, +-1e38)
//
// Replaces the reference's Triton kernel _ker_lm2exp (triturus/lm2exp.py:63-164) with one persistent,
// warp-specialised sm_100a kernel.  As a GEMM: D[M = i, N = k] = A[M, Kc = j] * B[Kc, N].
//
//   warp 0      TMA producer: a-tiles (128 x 32 fp32, K-major, 128B swizzle) into the operand ring and raw
//               b-tiles (32 j-rows x BN k-columns, dense) into the raw ring.
//   warp 1      allocates TMEM; one lane issues tcgen05.mma.kind::tf32 (M = 128, N = BN, K = 8) and commits.
//   warps 4-7   epilogue: tcgen05.ld the fp32 accumulator, out = m + log(acc), 128-bit stores.
//   warps 8+    transform: raw b -> exp(b - m) in registers -> tf32-rounded K-major swizzled B operand.
//
// One CTA tile is (MT * 128) rows x BN columns; the MT row blocks share each generated B operand, so one
// exp feeds MT * 128 MACs.  Accumulators live in TMEM (MT * BN columns per buffer, double-buffered when
// 2 * MT * BN <= 512) so the epilogue of one tile overlaps the main loop of the next.
//
// PREC = 1 selects the 3xTF32 split: a = a_hi + a_lo, e = e_hi + e_lo and
// acc += a_hi*e_lo + a_lo*e_hi + a_hi*e_hi, which restores ~fp32 accuracy at a third of the MMA rate.
#pragma once

#include "ptx.cuh"

namespace tb200 {

struct Lm2expParams {
  const float* m_ws;   // [R, K] clamped column maxima of b
  float* out;          // [R, I, K]
  int64_t out_s0, out_s1;  // element strides of out (innermost stride is 1)
  int R, I, J, K;
  int tiles_m, tiles_n, num_tiles;
  int* status;
};

template <int BN_, int MT_, int PREC_, int NS_, int NR_, int NTW_>
struct Lm2expCfg {
  static constexpr int BM = 128, BK = 32;
  static constexpr int BN = BN_, MT = MT_, PREC = PREC_, NS = NS_, NR = NR_, NTW = NTW_;
  static constexpr int NCOPY = PREC ? 2 : 1;               // hi (+ lo) copies of each operand
  static constexpr int A_TILE = BM * BK * 4;               // 16 KB
  static constexpr int B_TILE = BN * BK * 4;
  static constexpr int STAGE = NCOPY * (MT * A_TILE + B_TILE);
  static constexpr int RAW = BK * BN * 4;
  static constexpr int ACC_COLS = MT * BN;
  static constexpr int NBUF = (2 * ACC_COLS <= 512) ? 2 : 1;
  static constexpr int TMEM_COLS = (NBUF * ACC_COLS <= 128) ? 128 : (NBUF * ACC_COLS <= 256 ? 256 : 512);
  static constexpr int NTHREADS = (8 + NTW) * 32;
  static constexpr int NTT = NTW * 32;                     // transform threads
  static constexpr int THR_PER_COL = NTT / BN;             // transform threads sharing one column
  static constexpr int GROUPS = 8 / THR_PER_COL;           // groups of 4 j-rows per thread per k-block
  static constexpr int NBAR = 3 * NS + 2 * NR + 4;
  static constexpr int SMEM_BYTES = 1024 /*align slack*/ + NS * STAGE + NR * RAW + NBAR * 8 + 64;
  static_assert(NTT % BN == 0 && (8 % THR_PER_COL) == 0 && THR_PER_COL >= 1, "transform thread mapping");
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "BN");
  static_assert(NBUF * ACC_COLS <= 512, "TMEM capacity");
  static_assert(SMEM_BYTES <= 232448, "shared memory capacity");
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
lm2exp_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
              const Lm2expParams p) {
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, MT = Cfg::MT, NS = Cfg::NS, NR = Cfg::NR;
  constexpr int PREC = Cfg::PREC, NTW = Cfg::NTW;

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128B-swizzled operand tiles.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;                              // NS stages of [A copies | B copies]
  uint8_t* raw_base = smem + NS * Cfg::STAGE;              // NR raw b tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(raw_base + NR * Cfg::RAW);
  uint64_t* a_full = bars;                 // [NS] TMA bytes of the a-tiles landed
  uint64_t* b_full = bars + NS;            // [NS] transform warps finished the B operand (and a split)
  uint64_t* opnd_empty = bars + 2 * NS;    // [NS] MMAs reading the stage retired
  uint64_t* raw_full = bars + 3 * NS;      // [NR] TMA bytes of the raw b-tile landed
  uint64_t* raw_empty = raw_full + NR;     // [NR] transform warps done reading the raw tile
  uint64_t* acc_full = raw_empty + NR;     // [2] accumulator buffer complete
  uint64_t* acc_empty = acc_full + 2;      // [2] epilogue drained the buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
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
      mbar_init(&a_full[s], 1);
      mbar_init(&b_full[s], NTW);
      mbar_init(&opnd_empty[s], 1);
    }
    for (int s = 0; s < NR; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], NTW);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 4);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int KB = (p.J + BK - 1) / BK;  // k-blocks per tile

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
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % NS;
          const uint32_t ph = (it / NS) & 1;
          if (!(ok = mbar_wait(&opnd_empty[s], ph ^ 1, ctl, STATUS_TIMEOUT_PRODUCER))) break;
          mbar_arrive_expect_tx(&a_full[s], MT * Cfg::A_TILE);
#pragma unroll
          for (int t = 0; t < MT; ++t) tma_load_3d(a_tile(s, 0, t), &tmap_a, &a_full[s], kb * BK, i0 + t * BM, r);
          const int rs = it % NR;
          const uint32_t rph = (it / NR) & 1;
          if (!(ok = mbar_wait(&raw_empty[rs], rph ^ 1, ctl, STATUS_TIMEOUT_PRODUCER))) break;
          mbar_arrive_expect_tx(&raw_full[rs], Cfg::RAW);
          tma_load_3d(raw_base + rs * Cfg::RAW, &tmap_b, &raw_full[rs], n0, kb * BK, r);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(BM, BN);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcount) {
        const int buf = tcount % Cfg::NBUF;
        const uint32_t aph = (tcount / Cfg::NBUF) & 1;
        if (!(ok = mbar_wait(&acc_empty[buf], aph ^ 1, ctl, STATUS_TIMEOUT_MMA))) break;
        tc_fence_after_sync();
        for (int kb = 0; kb < KB; ++kb, ++it) {
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
              const uint32_t acc = (kb > 0 || ks > 0) ? 1u : 0u;
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
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const bool vec_ok = ((p.K & 3) == 0) && ((p.out_s1 & 3) == 0) && ((p.out_s0 & 3) == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcount) {
      int r, n0, i0;
      decode(tile, r, n0, i0);
      const int buf = tcount % Cfg::NBUF;
      const uint32_t aph = (tcount / Cfg::NBUF) & 1;
      if (!(ok = mbar_wait_warp(&acc_full[buf], aph, ctl, STATUS_TIMEOUT_EPILOGUE))) break;
      tc_fence_after_sync();
#pragma unroll 1
      for (int t = 0; t < MT; ++t) {
        if (i0 + t * BM >= p.I) break;  // whole row block is padding
        const int row = i0 + t * BM + q * 32 + lane;
        float* out_row = p.out + static_cast<int64_t>(r) * p.out_s0 + static_cast<int64_t>(row) * p.out_s1;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int k0 = n0 + c * 32;
          if (k0 >= p.K) break;  // whole chunk is padding
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * Cfg::ACC_COLS + t * BN + c * 32, v);
          const float m_lane = (k0 + lane < p.K) ? __ldg(p.m_ws + static_cast<int64_t>(r) * p.K + k0 + lane) : 0.f;
          tmem_ld_wait();
          float o[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const float m_e = __shfl_sync(0xffffffffu, m_lane, e);
            const float acc = __uint_as_float(v[e]);
            o[e] = m_e + (PREC ? logf(acc) : lg2_approx(acc) * LN2_F);
          }
          if (row < p.I) {
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
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ transform: raw b -> B operand
    const int tt = threadIdx.x - 8 * 32;
    const int n = tt % BN;                         // column of the tile owned by this thread
    const int g0 = (tt / BN) * Cfg::GROUPS;        // first group of 4 j-rows owned by this thread
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
      int r, n0, i0;
      decode(tile, r, n0, i0);
      const int kcol = n0 + n;
      const float m_n = (kcol < p.K) ? __ldg(p.m_ws + static_cast<int64_t>(r) * p.K + kcol) : 0.f;
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int s = it % NS;
        const uint32_t ph = (it / NS) & 1;
        const int rs = it % NR;
        const uint32_t rph = (it / NR) & 1;
        if (!(ok = mbar_wait_warp(&raw_full[rs], rph, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
        if (!(ok = mbar_wait_warp(&opnd_empty[s], ph ^ 1, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
        const float* raw = reinterpret_cast<const float*>(raw_base + rs * Cfg::RAW);
        uint8_t* bh = b_tile(s, 0);
        uint8_t* bl = b_tile(s, PREC ? 1 : 0);
        const int jrem = p.J - kb * BK;  // rows of this k-block that exist (>= 32 except in the tail)
#pragma unroll
        for (int gg = 0; gg < Cfg::GROUPS; ++gg) {
          const int g = g0 + gg;
          float e[4];
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int jj = g * 4 + x;
            const float v = raw[jj * BN + n];
            // Rows past J and columns past K must be exact zeros in the operand: the TMA zero fill is
            // in log space, and exp(0 - m) is not zero.
            e[x] = (jj < jrem && kcol < p.K) ? exp_shifted(v, m_n) : 0.f;
          }
          const uint32_t off = static_cast<uint32_t>(n) * 128u + ((static_cast<uint32_t>(g) ^ (n & 7u)) << 4);
          if (PREC) {
            float hi[4], lo[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) tf32_split_rn(e[x], hi[x], lo[x]);
            *reinterpret_cast<float4*>(bh + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<float4*>(bl + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
          } else {
            uint4 w;
            w.x = tf32_round_bits(e[0]);
            w.y = tf32_round_bits(e[1]);
            w.z = tf32_round_bits(e[2]);
            w.w = tf32_round_bits(e[3]);
            *reinterpret_cast<uint4*>(bh + off) = w;
          }
        }
        if (PREC) {
          // Split the a-tiles in place: hi keeps the tf32 bits, lo = a - hi goes to the second copy.
          if (!(ok = mbar_wait_warp(&a_full[s], ph, ctl, STATUS_TIMEOUT_TRANSFORM))) break;
          float4* ah = reinterpret_cast<float4*>(a_tile(s, 0, 0));
          float4* al = reinterpret_cast<float4*>(a_tile(s, 1, 0));
          for (int c = tt; c < MT * Cfg::A_TILE / 16; c += Cfg::NTT) {
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
        if (lane == 0) {
          mbar_arrive(&b_full[s]);
          mbar_arrive(&raw_empty[rs]);
        }
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
}

}  // namespace tb200
