// extern "C" boundary of libtriturus_b200.so: argument validation, tensor-map encoding, tile-shape
// selection and kernel launches.  Declarations and the reference interfaces they replace are in
// include/triturus_b200.h.  Nothing here allocates device memory or synchronises.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include <cstring>
#include <mutex>

#include "../../include/triturus_b200.h"
#include "lm2exp_kernel.cuh"
#include "lm2exp_pair_kernel.cuh"
#include "lm2exp_tspair_kernel.cuh"
#include "lt2exp_kernel.cuh"
#include "lt2exp_tmem_kernel.cuh"

namespace tb200 {

// ----------------------------------------------------------------------------- stabiliser pre-pass

// m[r,k] = clamp(max_j x[r,j,k]).  One block owns 32 columns of one batch entry; its 8 warps split the
// rows.  In the vector path a warp reads 4 rows x 128 bytes per step (lane = 4 * row + float4 group) and
// folds the four row slots with warp shuffles.
template <bool VEC>
__global__ void __launch_bounds__(256) colmax_kernel(const float* __restrict__ x, float* __restrict__ m, int J, int K,
                                                      int64_t s0, int64_t s1, int64_t s2, int R, const int* only_if,
                                                      int* publish) {
  __shared__ float part[8][32];
  // The contraction kernel that consumes m may be launched as a programmatic dependent: let it start its set-up
  // (barriers, tensor memory, first operand tiles) as soon as every block of this grid is running.
  pdl_launch_dependents();
  // A conditional launch (the exact pass behind an optimistic contraction, launched as that kernel's programmatic
  // dependent) waits for it and does nothing unless it raised the flag.
  // Block 0 republishes the decision in a second word for the conditional contraction behind this launch, so
  // that that kernel can put the flag itself down again without a reader still being out.
  if (only_if != nullptr) {
    pdl_wait();
    const bool up = *only_if != 0;
    if (blockIdx.x == 0 && threadIdx.x == 0) *publish = up ? 1 : 0;
    if (!up) return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Work items (32-column block, batch entry) are walked with a grid stride: an ordinary launch has one block per
  // item, a conditional one a few blocks per SM (thousands of blocks that only read the flag and leave would
  // cost tens of microseconds on every call).
  const int nbx = (K + 31) / 32;
  const int64_t items = static_cast<int64_t>(nbx) * R;
  for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
  const int r = static_cast<int>(item / nbx);
  const int c0 = static_cast<int>(item % nbx) * 32;
  const float* xb = x + static_cast<int64_t>(r) * s0;
  if (VEC) {
    const int cg = lane & 7, rs = lane >> 3;
    const int c = c0 + cg * 4;
    float4 mx = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    if (c < K) {  // K % 4 == 0 in this path, so the float4 is entirely inside the row
      for (int j = warp * 4 + rs; j < J; j += 32) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(xb + static_cast<int64_t>(j) * s1 + c));
        mx.x = fmaxf(mx.x, v.x);
        mx.y = fmaxf(mx.y, v.y);
        mx.z = fmaxf(mx.z, v.z);
        mx.w = fmaxf(mx.w, v.w);
      }
    }
#pragma unroll
    for (int sh = 8; sh <= 16; sh <<= 1) {
      mx.x = fmaxf(mx.x, __shfl_xor_sync(0xffffffffu, mx.x, sh));
      mx.y = fmaxf(mx.y, __shfl_xor_sync(0xffffffffu, mx.y, sh));
      mx.z = fmaxf(mx.z, __shfl_xor_sync(0xffffffffu, mx.z, sh));
      mx.w = fmaxf(mx.w, __shfl_xor_sync(0xffffffffu, mx.w, sh));
    }
    if (rs == 0) {
      part[warp][cg * 4 + 0] = mx.x;
      part[warp][cg * 4 + 1] = mx.y;
      part[warp][cg * 4 + 2] = mx.z;
      part[warp][cg * 4 + 3] = mx.w;
    }
  } else {
    const int c = c0 + lane;
    float mx = -INFINITY;
    if (c < K) {
      for (int j = warp; j < J; j += 8) mx = fmaxf(mx, __ldg(xb + static_cast<int64_t>(j) * s1 + c * s2));
    }
    part[warp][lane] = mx;
  }
  __syncthreads();
  if (warp == 0) {
    float mx = part[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, part[w][lane]);
    const int c = c0 + lane;
    if (c < K) m[static_cast<int64_t>(r) * K + c] = clamp_stab(mx);
  }
  __syncthreads();  // `part` is rewritten by the next item
  }
}

// The same stabiliser for a b stored with j contiguous (a transposed view): m[r,k] = clamp(max_j x[r,k,j]), one warp
// per row of J consecutive values, eight rows per block.
__global__ void __launch_bounds__(256) rowmax_kernel(const float* __restrict__ x, float* __restrict__ m, int J, int K,
                                                      int64_t s0, int64_t sk) {
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k = blockIdx.x * 8 + warp;
  const int r = blockIdx.y;
  if (k >= K) return;
  const float* row = x + static_cast<int64_t>(r) * s0 + static_cast<int64_t>(k) * sk;
  float mx = -INFINITY;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const int J4 = J & ~3;
    for (int j = lane * 4; j < J4; j += 128) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(row + j));
      mx = fmaxf(fmaxf(mx, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
    }
    for (int j = J4 + lane; j < J; j += 32) mx = fmaxf(mx, __ldg(row + j));
  } else {
    for (int j = lane; j < J; j += 32) mx = fmaxf(mx, __ldg(row + j));
  }
#pragma unroll
  for (int sh = 16; sh >= 1; sh >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
  if (lane == 0) m[static_cast<int64_t>(r) * K + k] = clamp_stab(mx);
}

// Fills m[0..n) with -inf: the start value of the column maxima that an epilogue folds into it.
__global__ void __launch_bounds__(256) fill_neg_inf_kernel(float* __restrict__ m, int64_t n) {
  for (int64_t i = blockIdx.x * 256 + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * 256) m[i] = -INFINITY;
}

// Self-test of the failure path every kernel of this library shares: warp 1 waits on an mbarrier on which
// nobody ever arrives, with a wait limit of `limit_cycles`; the wait gives up, raises the CTA's abort flag and
// writes its code to the status word; warp 0, waiting on a second barrier with the long production limit,
// sees the flag and leaves too; both warps meet at the final barrier and the kernel returns.  Nothing traps and
// nothing spins without a bound.
__global__ void __launch_bounds__(64) wait_timeout_selftest_kernel(int* status, long long limit_cycles) {
  __shared__ uint64_t never[2];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(&never[0], 1);
    mbar_init(&never[1], 1);
    fence_mbar_init();
  }
  __syncthreads();
  const AbortCtl ctl{abort_flag, status};
  const int warp = threadIdx.x >> 5;
  if (warp == 1) {
    mbar_wait_warp(&never[0], 0, ctl, STATUS_TIMEOUT_SETUP, limit_cycles);
  } else {
    mbar_wait_warp(&never[1], 0, ctl, STATUS_TIMEOUT_EPILOGUE);
  }
  __syncthreads();
}

// ----------------------------------------------------------------------------- driver entry point for tensor maps

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

// fp32 tensor map of rank `rank`; dims/strides listed innermost first, strides in elements
// (strides[0] is the innermost stride and must be 1).
static int make_tmap(CUtensorMap* out, const float* base, int rank, const int64_t* dims, const int64_t* strides,
                     const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return TRITURUS_B200_EDRIVER;
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5], es[5];
  for (int d = 0; d < rank; ++d) {
    gdim[d] = static_cast<cuuint64_t>(dims[d]);
    bx[d] = box[d];
    es[d] = 1;
    if (d > 0) gstr[d - 1] = static_cast<cuuint64_t>(strides[d]) * sizeof(float);
  }
  const CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, static_cast<cuuint32_t>(rank),
                         const_cast<float*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? TRITURUS_B200_OK : TRITURUS_B200_ETENSORMAP;
}

static int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// A stride is usable by TMA when it is a positive multiple of 4 elements; strides of size-1 dimensions
// are irrelevant and get a safe value instead.
static bool fix_stride(int64_t size, int64_t& stride, int64_t natural) {
  if (size == 1) {
    stride = natural;
    return true;
  }
  return stride > 0 && (stride & 3) == 0;
}

static int64_t round_up4(int64_t v) { return (v + 3) & ~int64_t(3); }

// ----------------------------------------------------------------------------- lm2exp launch

// `after_prepass`: the stabiliser pre-pass was launched just before on the same stream; the kernel is then
// launched as its programmatic dependent (its threads wait for the pre-pass before they read m).
template <class Kern, class... Args>
static int launch_maybe_dependent(Kern kern, dim3 grid, int threads, int smem, cudaStream_t stream, bool after_prepass,
                                  Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = after_prepass ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...) == cudaSuccess ? TRITURUS_B200_OK : TRITURUS_B200_ELAUNCH;
}

template <class Cfg>
static int launch_lm2exp(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, Lm2expParams p,
                         cudaStream_t stream, bool after_prepass) {
  auto kern = lm2exp_kernel<Cfg>;
  static std::once_flag once[64];
  static cudaError_t attr_rc[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return TRITURUS_B200_ELAUNCH;
  std::call_once(once[dev], [&] {
    attr_rc[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  });
  if (attr_rc[dev] != cudaSuccess) return TRITURUS_B200_ELAUNCH;
  p.tiles_m = (p.I + Cfg::BM * Cfg::MT - 1) / (Cfg::BM * Cfg::MT);
  p.tiles_n = (p.K + Cfg::BN - 1) / Cfg::BN;
  const int64_t nt = static_cast<int64_t>(p.R) * p.tiles_m * p.tiles_n;
  if (nt > INT32_MAX) return TRITURUS_B200_EINVAL;
  p.num_tiles = static_cast<int>(nt);
  const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  return launch_maybe_dependent(kern, dim3(static_cast<unsigned>(grid)), Cfg::NTHREADS, Cfg::SMEM_BYTES, stream, after_prepass, ta,
                                tb, to, p);
}

//                          BN   MT PREC NS
using LmT_128_1 = Lm2expCfg<128, 1, 0, 6>;
using LmT_128_2 = Lm2expCfg<128, 2, 0, 4>;
using LmT_256_1 = Lm2expCfg<256, 1, 0, 4>;
using LmT_256_2 = Lm2expCfg<256, 2, 0, 3>;
using LmX_128_1 = Lm2expCfg<128, 1, 1, 3>;
using LmX_128_2 = Lm2expCfg<128, 2, 1, 2>;

// plain TF32 with chunked re-summation of the accumulator, for contractions of more than 32 K terms
using LmP_128_1 = Lm2expCfg<128, 1, 0, 6, true>;
using LmP_128_2 = Lm2expCfg<128, 2, 0, 4, true>;

// the same tiles with the paths for a transposed b and for operands fetched element by element
using LmTo_128_1 = Lm2expCfg<128, 1, 0, 6, false, false, true>;
using LmTo_128_2 = Lm2expCfg<128, 2, 0, 4, false, false, true>;
using LmTo_256_1 = Lm2expCfg<256, 1, 0, 4, false, false, true>;
using LmTo_256_2 = Lm2expCfg<256, 2, 0, 3, false, false, true>;
using LmXo_128_1 = Lm2expCfg<128, 1, 1, 3, true, false, true>;
using LmXo_128_2 = Lm2expCfg<128, 2, 1, 2, true, false, true>;
using LmPo_128_1 = Lm2expCfg<128, 1, 0, 6, true, false, true>;
using LmPo_128_2 = Lm2expCfg<128, 2, 0, 4, true, false, true>;

// plain matrix product (the reference's mm): 256 x 128 tiles, no stabiliser / exp / log
using LmPlainT = Lm2expCfg<128, 2, 0, 4, false, true>;
using LmPlainX = Lm2expCfg<128, 2, 1, 2, true, true>;

using LmPairT = Lm2expPairCfg<0, 6>;
using LmPairX = Lm2expPairCfg<1, 3>;

// Launch on CTA pairs: a cluster of two CTAs per 256 x 256 tile.
template <class Cfg>
static int launch_lm2exp_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, Lm2expParams p,
                              cudaStream_t stream, bool after_prepass) {
  auto kern = lm2exp_pair_kernel<Cfg>;
  static std::once_flag once[64];
  static cudaError_t attr_rc[64];
  static int max_clusters[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return TRITURUS_B200_ELAUNCH;
  std::call_once(once[dev], [&] {
    attr_rc[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    max_clusters[dev] = sm_count() / 2;
    if (attr_rc[dev] == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(sm_count() & ~1), 1, 1);
      cfg.blockDim = dim3(Cfg::NTHREADS, 1, 1);
      cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2;
      at[0].val.clusterDim.y = 1;
      at[0].val.clusterDim.z = 1;
      cfg.attrs = at;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) max_clusters[dev] = n;
    }
  });
  if (attr_rc[dev] != cudaSuccess) return TRITURUS_B200_ELAUNCH;
  p.tiles_m = (p.I + 2 * Cfg::BM - 1) / (2 * Cfg::BM);
  p.tiles_n = (p.K + Cfg::BN - 1) / Cfg::BN;
  const int64_t nt = static_cast<int64_t>(p.R) * p.tiles_m * p.tiles_n;
  if (nt > INT32_MAX) return TRITURUS_B200_EINVAL;
  p.num_tiles = static_cast<int>(nt);
  const int clusters = p.num_tiles < max_clusters[dev] ? p.num_tiles : max_clusters[dev];
  return launch_maybe_dependent(kern, dim3(static_cast<unsigned>(2 * clusters)), Cfg::NTHREADS, Cfg::SMEM_BYTES, stream,
                                after_prepass, ta, tb, to, p);
}

//                                  NS NSB groups optimistic
using LmTsPair = Lm2expTsPairCfg<8, 4, 2>;
using LmTsPairOpt = Lm2expTsPairCfg<8, 4, 2, true>;
using LmTsPairFused = Lm2expTsPairCfg<8, 4, 2, false, true>;  // exact max pass inside: the conditional launch behind Opt

// The CTA-pair kernel with the generated operand in tensor memory (plain TF32, a with j contiguous).
template <class Cfg>
static int launch_lm2exp_tspair(const CUtensorMap& ta, const CUtensorMap& tb_plain, const CUtensorMap& to,
                                Lm2expParams p, cudaStream_t stream, bool after_prepass) {
  auto kern = lm2exp_tspair_kernel<Cfg>;
  static std::once_flag once[64];
  static cudaError_t attr_rc[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return TRITURUS_B200_ELAUNCH;
  std::call_once(once[dev], [&] {
    attr_rc[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  });
  if (attr_rc[dev] != cudaSuccess) return TRITURUS_B200_ELAUNCH;
  p.tiles_m = (p.I + Cfg::BN - 1) / Cfg::BN;
  p.tiles_n = (p.K + 2 * Cfg::BM - 1) / (2 * Cfg::BM);
  const int64_t nt = static_cast<int64_t>(p.R) * p.tiles_m * p.tiles_n;
  if (nt > INT32_MAX) return TRITURUS_B200_EINVAL;
  p.num_tiles = static_cast<int>(nt);
  const int max_clusters = sm_count() / 2;  // one CTA per SM (shared memory and all of TMEM), pairs on SM pairs
  const int clusters = p.num_tiles < max_clusters ? p.num_tiles : max_clusters;
  return launch_maybe_dependent(kern, dim3(static_cast<unsigned>(2 * clusters)), Cfg::NTHREADS, Cfg::SMEM_BYTES, stream,
                                after_prepass, ta, tb_plain, to, p);
}

static int64_t tile_count(int64_t R, int64_t rows, int64_t cols, int bn, int mt) {
  return R * ((rows + 128 * mt - 1) / (128 * mt)) * ((cols + bn - 1) / bn);
}

// Tile shape with the smallest estimated run time: waves x tile work x shared-memory cycles per tensor cycle.
// All kernels are bound by the shared-memory pipe, and a larger tile moves fewer bytes through it per MAC
// (the factors are bytes per k-block / 128 B per clock over the k-block's tensor cycles), so a larger tile
// wins unless it leaves the last wave mostly empty.
static int auto_variant(int64_t R, int64_t rows, int64_t cols, bool allow_bn256, bool in_place_transform,
                        int max_acc_cols = 512) {
  const int sms = sm_count();
  const int mt_max = rows > 128 ? 2 : 1;
  const int bn_max = (cols > 128 && allow_bn256) ? 256 : 128;
  int best = 1281;
  double best_cost = 1e300;
  for (int bn = 128; bn <= bn_max; bn *= 2) {
    for (int mt = 1; mt <= mt_max; ++mt) {
      if (mt * bn > max_acc_cols) continue;  // the caller needs TMEM columns beside the accumulator
      const int64_t waves = (tile_count(R, rows, cols, bn, mt) + sms - 1) / sms;
      // per k-block: a-tiles in + operand read, b in (+ read + write back when transformed in place),
      // operand read of b once per row block
      const double kb_bytes = mt * 16384.0 * 2 + bn * 128.0 * (in_place_transform ? 3 : 1) + bn * 128.0 * mt;
      const double tensor_cycles = mt * bn * 2.0;  // 128 x bn x 32 MACs at 2048 per clock
      const double factor = (kb_bytes / 128.0) / tensor_cycles;
      const double cost = static_cast<double>(waves) * mt * bn * (factor > 1.0 ? factor : 1.0);
      if (cost < best_cost) {
        best_cost = cost;
        best = bn * 10 + mt;
      }
    }
  }
  return best;
}

// What a call of triturus_b200_lm2exp_f32 will run for a problem size, precision and variant code.
struct Lm2expPlan {
  int bn, mt;   // output columns per tile, 128-row blocks per CTA
  bool pair;    // 256 x 256 tile on a pair of CTAs
  bool tspair;  // ... by the kernel that keeps the generated operand in tensor memory (variants 2566, 2567)
  bool optimistic;  // ... without a pre-pass: stabiliser from the first k-block, exact passes as conditional launches (2567)
  bool fused;   // max pass inside the contraction kernel (no pre-pass launch)
  bool optimistic_fused;  // ... over the first k-block of each slab only, exact pass as a conditional launch
  bool optimistic_prepass;  // pair tile in shared memory: pre-pass over the first 32 rows, exact passes conditional
  bool colmax_exclusive;  // one row tile covers I: column maxima of the result are stored, not reduced
  bool promote_tf32;      // plain TF32 over more than kLongContraction terms: accumulator re-summed in chunks
};

// Contractions longer than this run with the chunked re-summation of the accumulator in plain TF32 too: the
// tensor core's truncating adds lose ~1.5e-8 per term (2.6e-4 in log space at 16 K terms, 2.5e-3 at 256 K).
constexpr int64_t kLongContraction = 32768;

// have_m: the caller supplies the stabiliser, so the tile is chosen as usual but no max pass of either kind runs.
// b_km: b is stored with j contiguous; only the single-CTA kernel takes it, with the pre-pass stabiliser.
// single_cta: an operand is fetched element by element, which only the single-CTA kernel does.
static int plan_lm2exp(int64_t R, int64_t I, int64_t J, int64_t K, int precision, int variant, Lm2expPlan* out,
                       bool have_m = false, bool b_km = false, bool single_cta = false) {
  if (variant < 0) return TRITURUS_B200_EINVAL;
  // 0 = automatic, 1 = pre-pass, 2 = fused max pass, 3 = fused max pass over the first k-block only (optimistic),
  // 4 = pre-pass over the first 32 rows only (optimistic; shared-memory pair tile)
  const int stab_mode = variant / 100000;
  int tile_variant = variant % 100000;
  if (stab_mode > 4 || (have_m && stab_mode >= 2)) return TRITURUS_B200_EINVAL;
  if (tile_variant == 0) {
    // More than one 256-row tile per column slab: the stabiliser comes from a pre-pass anyway, and a CTA
    // pair moves the fewest shared-memory bytes per MAC.  With the optimistic stabilisers, which need no full
    // pre-pass, the pair kernels also win from two 128-row blocks on (cfg3, I = 256: 0.479 ms on the
    // TMEM-operand pair kernel against 0.508 ms on the single-CTA kernel with the optimistic fused max pass; in
    // 3xTF32 1.14 against 1.30 ms).  Otherwise a single-CTA tile with the fused max pass.
    // (Not for 3xTF32 contractions longer than 4096, where the drift of the tensor core's truncating
    // accumulator, ~1.2e-8 per term, would use up the 3xTF32 tolerance: only the single-CTA kernel re-sums
    // its accumulator in chunks.)
    // The optimistic forms cost two or three launches more, which return at once on the device but take the host
    // some 7 us per call: below ~50 us of work a loop of calls would wait for the host (R64 256^3: 14.4 us per
    // call on the device but 24 us in an eager loop, against 18.3 / 17.7 us for the single launch).
    const bool big = 2.0 * static_cast<double>(R) * I * J * K >= 2e10;
    const bool long_3x = precision == TRITURUS_B200_PRECISION_3XTF32 && J > 4096;
    const bool long_tf = precision == TRITURUS_B200_PRECISION_TF32 && J > kLongContraction;
    const bool want_pair = !b_km && !single_cta && (stab_mode < 2 || stab_mode == 4) && !long_3x && !long_tf &&
                           (I > 256 || (I > 128 && J >= 128 && !have_m && stab_mode != 1 && big)) && K > 128 &&
                           tile_count(R, I, K, 256, 2) >= sm_count() / 4;
    // (long plain-TF32 contractions: 128 columns, so that the master copy fits beside the accumulator)
    // Plain TF32 on pairs: the TMEM-operand kernel, with the optimistic stabiliser unless a pre-pass was asked for.
    const int pair_variant = precision != TRITURUS_B200_PRECISION_TF32 || stab_mode == 4 ? 2564
                             : (stab_mode == 0 && !have_m && big ? 2567 : 2566);
    if (stab_mode == 4 && !want_pair) return TRITURUS_B200_EINVAL;
    tile_variant = want_pair ? pair_variant : auto_variant(R, I, K, precision == TRITURUS_B200_PRECISION_TF32 && !long_tf, true);
  }
  if (b_km && (tile_variant == 2564 || tile_variant == 2566 || tile_variant == 2567 || stab_mode >= 2))
    return TRITURUS_B200_EINVAL;
  if (single_cta && (tile_variant == 2564 || tile_variant == 2566 || tile_variant == 2567)) return TRITURUS_B200_EINVAL;
  const bool optimistic = tile_variant == 2567 && stab_mode == 0 && !have_m;
  const bool tspair = tile_variant == 2566 || tile_variant == 2567;
  if (tspair) {
    if (precision != TRITURUS_B200_PRECISION_TF32) return TRITURUS_B200_EINVAL;
    tile_variant = 2564;  // same tile and stabiliser handling as the other CTA-pair kernel
  }
  int bn = tile_variant / 10;
  const int mt = tile_variant % 10;
  const bool pair = tile_variant == 2564;  // 256 x 256 tile on a pair of CTAs, 128 rows each
  if (!pair && ((bn != 128 && bn != 256) || (mt != 1 && mt != 2))) return TRITURUS_B200_EINVAL;
  if (pair && (stab_mode == 2 || stab_mode == 3)) return TRITURUS_B200_EINVAL;  // the pair kernels take m from a pre-pass
  if (stab_mode == 4 && (!pair || tspair)) return TRITURUS_B200_EINVAL;
  if (!pair && precision == TRITURUS_B200_PRECISION_3XTF32) bn = 128;  // hi/lo copies leave room for 128 columns
  // Fused max pass when every column slab of b feeds a single row tile: b then crosses HBM once.  Also when
  // the whole problem is less than one wave of tiles: a second launch then costs more than the row tiles of a
  // slab each scanning it (cfg1: 18.5 us against 21.7 us).
  const bool one_wave = tile_count(R, I, K, bn, mt) <= sm_count();
  const bool fused = !pair && !b_km && (stab_mode == 2 || stab_mode == 3 || (stab_mode == 0 && (I <= 128 * mt || one_wave)));
  // Such shapes are bound by HBM and by the epilogue: prefer 128 columns, whose accumulator is
  // double-buffered so that the epilogue overlaps the next tile.
  if (fused && variant % 100000 == 0 && bn == 256 && tile_count(R, I, K, 128, mt) >= sm_count()) bn = 128;
  out->bn = bn;
  out->mt = pair ? 4 : mt;
  out->pair = pair;
  out->tspair = tspair;
  out->optimistic = optimistic;
  out->fused = fused && !have_m;
  // Automatic: where the max pass is a real share of the work (four k-blocks or more) and the launch is long
  // enough (more than one wave of tiles) for two more, empty, launches not to matter.
  // Plain TF32 only: in 3xTF32 the shapes concerned are bound by the three MMAs per k-step, not by the max pass
  // (cfg3: 1.35 ms with, 1.32 ms without).
  const bool big_enough = 2.0 * static_cast<double>(R) * I * J * K >= 2e10;  // (see `big` above)
  out->optimistic_fused =
      out->fused && (stab_mode == 3 || (stab_mode == 0 && precision == TRITURUS_B200_PRECISION_TF32 && J >= 128 &&
                                        big_enough && tile_count(R, I, K, bn, mt) > sm_count()));
  out->colmax_exclusive = !pair && I <= 128 * mt;
  // The shared-memory pair kernel, where it is the automatic choice (3xTF32): the pre-pass scans 32 rows instead of J.
  out->optimistic_prepass = pair && !tspair && !have_m && J >= 128 &&
                            (stab_mode == 4 || (stab_mode == 0 && variant % 100000 == 0 && big_enough));
  out->promote_tf32 = !pair && bn == 128 && precision == TRITURUS_B200_PRECISION_TF32 && J > kLongContraction;
  return TRITURUS_B200_OK;
}

}  // namespace tb200

using namespace tb200;

extern "C" {

#ifdef TB200_TIMELINE
// Development builds only: copy the timeline of the last launch of the TMEM-operand pair kernel to the host.
int triturus_b200_debug_timeline(long long* host, int n) {
  return cudaMemcpyFromSymbol(host, tb200::g_timeline, sizeof(long long) * n) == cudaSuccess ? 0 : -1;
}
#endif

int triturus_b200_version(void) { return 100; }

const char* triturus_b200_strerror(int code) {
  switch (code) {
    case TRITURUS_B200_OK: return "ok";
    case TRITURUS_B200_EINVAL: return "invalid argument (shape, pointer, precision or variant)";
    case TRITURUS_B200_EALIGN: return "pointer or stride violates the 16-byte alignment rules";
    case TRITURUS_B200_EWORKSPACE: return "workspace too small or misaligned";
    case TRITURUS_B200_ETENSORMAP: return "tensor map rejected by the driver";
    case TRITURUS_B200_ELAUNCH: return "kernel launch failed";
    case TRITURUS_B200_EDRIVER: return "cuTensorMapEncodeTiled unavailable";
    case TRITURUS_B200_ESTATICLIMIT: return "R * K exceeds the built-in scratch of the static entry point";
    case STATUS_TIMEOUT_PRODUCER: return "device: TMA producer wait timed out";
    case STATUS_TIMEOUT_TRANSFORM: return "device: transform warp wait timed out";
    case STATUS_TIMEOUT_MMA: return "device: MMA issuer wait timed out";
    case STATUS_TIMEOUT_EPILOGUE: return "device: epilogue wait timed out";
    case STATUS_TIMEOUT_SETUP: return "device: setup wait timed out";
    default: return "unknown code";
  }
}

int triturus_b200_selftest_wait_timeout(int32_t* status_dev, int64_t limit_cycles, void* stream) {
  // at most ~0.1 s of spinning: this is a test of the error path, not a way to occupy a GPU
  if (status_dev == nullptr || limit_cycles < 1000 || limit_cycles > 200000000LL) return TRITURUS_B200_EINVAL;
  wait_timeout_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status_dev, limit_cycles);
  return cudaGetLastError() == cudaSuccess ? TRITURUS_B200_OK : TRITURUS_B200_ELAUNCH;
}

static int colmax_run(const float* x, float* m, int64_t R, int64_t J, int64_t K, const int64_t x_strides[3],
                      void* stream, const int* only_if, int* publish) {
  if (x == nullptr || m == nullptr || x_strides == nullptr) return TRITURUS_B200_EINVAL;
  if (R <= 0 || J <= 0 || K <= 0 || J > INT32_MAX || K > INT32_MAX || R > INT32_MAX) return TRITURUS_B200_EINVAL;
  const int64_t s2 = K > 1 ? x_strides[2] : 1;
  const bool vec = s2 == 1 && (K & 3) == 0 && aligned16(x) && (x_strides[0] & 3) == 0 && (x_strides[1] & 3) == 0;
  const int64_t items = ((K + 31) / 32) * R;
  // (a conditional launch follows the optimistic contraction as its programmatic dependent, with few blocks)
  const bool dep = only_if != nullptr;
  const int64_t cap = dep ? static_cast<int64_t>(sm_count()) * 8 : static_cast<int64_t>(INT32_MAX);
  const dim3 grid(static_cast<unsigned>(items < cap ? items : cap));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int Ji = static_cast<int>(J), Ki = static_cast<int>(K), Ri = static_cast<int>(R);
  return vec ? launch_maybe_dependent(colmax_kernel<true>, grid, 256, 0, st, dep, x, m, Ji, Ki, x_strides[0], x_strides[1],
                                      s2, Ri, only_if, publish)
             : launch_maybe_dependent(colmax_kernel<false>, grid, 256, 0, st, dep, x, m, Ji, Ki, x_strides[0], x_strides[1],
                                      s2, Ri, only_if, publish);
}

int triturus_b200_colmax_f32(const float* x, float* m, int64_t R, int64_t J, int64_t K, const int64_t x_strides[3],
                             void* stream) {
  return colmax_run(x, m, R, J, K, x_strides, stream, nullptr, nullptr);
}

int triturus_b200_lm2exp_launches(int64_t R, int64_t I, int64_t J, int64_t K, int precision, int variant) {
  if (R <= 0 || I <= 0 || J <= 0 || K <= 0) return TRITURUS_B200_EINVAL;
  if (precision != TRITURUS_B200_PRECISION_TF32 && precision != TRITURUS_B200_PRECISION_3XTF32)
    return TRITURUS_B200_EINVAL;
  Lm2expPlan plan;
  const int rc = plan_lm2exp(R, I, J, K, precision, variant, &plan);
  if (rc != TRITURUS_B200_OK) return rc;
  // optimistic stabiliser: the contraction and the two conditional launches of the exact passes
  return plan.fused ? (plan.optimistic_fused ? 2 : 1) : (plan.optimistic_prepass ? 4 : 2);
}

int triturus_b200_lm2exp_plan(int64_t R, int64_t I, int64_t J, int64_t K, int precision, int variant) {
  if (R <= 0 || I <= 0 || J <= 0 || K <= 0) return TRITURUS_B200_EINVAL;
  if (precision != TRITURUS_B200_PRECISION_TF32 && precision != TRITURUS_B200_PRECISION_3XTF32)
    return TRITURUS_B200_EINVAL;
  Lm2expPlan plan;
  const int rc = plan_lm2exp(R, I, J, K, precision, variant, &plan);
  if (rc != TRITURUS_B200_OK) return rc;
  return (plan.fused ? (plan.optimistic_fused ? 3 : 2) : (plan.optimistic ? 0 : (plan.optimistic_prepass ? 4 : 1))) * 100000 +
         plan.bn * 10 +
         (plan.tspair ? (plan.optimistic ? 7 : 6) : plan.mt);
}

// Workspace layout: [two flag words of the optimistic stabiliser, padded to 256 bytes][R x K stabilisers].
// A workspace of only R * K floats (the layout before the flags existed) holds the stabilisers at offset 0.
constexpr size_t kLm2expFlagBytes = 256;

size_t triturus_b200_lm2exp_workspace_bytes(int64_t R, int64_t I, int64_t J, int64_t K) {
  (void)I;
  (void)J;
  if (R <= 0 || K <= 0) return 0;
  return kLm2expFlagBytes + static_cast<size_t>(R) * static_cast<size_t>(K) * sizeof(float);
}

// Shared body of the lm2exp entry points.  b_colmax (optional): [R, K] column maxima of b supplied by the
// caller, which replace the stabiliser pass.  out_colmax (optional): [R, K] receives max_i out[r, i, k].
static int lm2exp_run_block(const float* a, const float* b, float* out, int64_t R, int64_t I, int64_t J, int64_t K,
                      const int64_t a_strides[3], const int64_t b_strides[3], const int64_t out_strides[3],
                      int precision, int variant, const float* b_colmax, float* out_colmax, void* workspace,
                      size_t workspace_bytes, int32_t* status_dev, void* stream) {
  if (a == nullptr || b == nullptr || out == nullptr || a_strides == nullptr || b_strides == nullptr ||
      out_strides == nullptr)
    return TRITURUS_B200_EINVAL;
  if (R <= 0 || I <= 0 || J <= 0 || K <= 0) return TRITURUS_B200_EINVAL;
  if (R > 65535 || I > (1 << 30) || J > (1 << 30) || K > (1 << 30)) return TRITURUS_B200_EINVAL;
  if (precision != TRITURUS_B200_PRECISION_TF32 && precision != TRITURUS_B200_PRECISION_3XTF32)
    return TRITURUS_B200_EINVAL;
  if (b_colmax == nullptr &&
      (workspace == nullptr || workspace_bytes < static_cast<size_t>(R) * static_cast<size_t>(K) * sizeof(float) ||
       (reinterpret_cast<uintptr_t>(workspace) & 255) != 0))
    return TRITURUS_B200_EWORKSPACE;
  if (out_colmax != nullptr && (out_colmax == b_colmax || (reinterpret_cast<uintptr_t>(out_colmax) & 3) != 0))
    return TRITURUS_B200_EINVAL;

  int64_t as0 = a_strides[0], as1 = a_strides[1], as2 = a_strides[2];
  int64_t bs0 = b_strides[0], bs1 = b_strides[1], bs2 = b_strides[2];
  int64_t os0 = out_strides[0], os1 = out_strides[1], os2 = out_strides[2];
  if (K > 1 && os2 != 1) return TRITURUS_B200_EALIGN;
  if (I > 1 && os1 <= 0) return TRITURUS_B200_EALIGN;
  if (R > 1 && os0 <= 0) return TRITURUS_B200_EALIGN;
  if ((reinterpret_cast<uintptr_t>(a) & 3) != 0 || (reinterpret_cast<uintptr_t>(b) & 3) != 0) return TRITURUS_B200_EALIGN;
  // How each operand reaches shared memory.  a with j contiguous is a K-major tensor-core operand, a transposed
  // view (i contiguous) an MN-major one; b with k contiguous is MN-major, a transposed view (j contiguous)
  // K-major (single-CTA kernel only).  All four go through tensor maps when base and strides meet the TMA rules;
  // an operand that does not (row pitch not a multiple of 16 bytes, innermost stride other than 1, base not
  // 16-byte aligned) is fetched element by element by the single-CTA kernel instead (gen_a / gen_b).
  const int64_t as_raw[3] = {as0, as1, as2}, bs_raw[3] = {bs0, bs1, bs2};
  bool a_mn = J > 1 && as2 != 1;
  bool a_tma = aligned16(a);
  if (a_tma && a_mn) {
    a_tma = (I == 1 || as1 == 1) && fix_stride(J, as2, round_up4(I)) && fix_stride(R, as0, round_up4(I) * J);
  } else if (a_tma) {
    a_tma = fix_stride(I, as1, round_up4(J)) && fix_stride(R, as0, round_up4(J) * I);
  }
  bool b_km = K > 1 && bs2 != 1;
  bool b_tma = aligned16(b);
  if (b_tma && b_km) {
    b_tma = (J == 1 || bs1 == 1) && fix_stride(K, bs2, round_up4(J)) && fix_stride(R, bs0, round_up4(J) * K);
  } else if (b_tma) {
    b_tma = fix_stride(J, bs1, round_up4(K)) && fix_stride(R, bs0, round_up4(K) * J);
  }
  const bool gen_a = !a_tma, gen_b = !b_tma;
  if (gen_a) a_mn = false;
  if (gen_b) b_km = false;
  // (the element-wise loader takes the place of the warps that fold the column maxima of the result)
  if ((gen_a || gen_b) && out_colmax != nullptr) return TRITURUS_B200_EALIGN;

  Lm2expPlan plan;
  {
    // A supplied stabiliser makes every max pass redundant (and a fused max pass cannot be requested as well).
    const int prc = plan_lm2exp(R, I, J, K, precision, variant, &plan, b_colmax != nullptr, b_km, gen_a || gen_b);
    if (prc != TRITURUS_B200_OK) return prc;
  }
  const int bn = plan.bn, mt = plan.mt;
  const bool pair = plan.pair, fused = plan.fused;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t m_bytes = static_cast<size_t>(R) * static_cast<size_t>(K) * sizeof(float);
  const bool ws_flags = workspace != nullptr && workspace_bytes >= kLm2expFlagBytes + m_bytes;
  float* m_buf = ws_flags ? reinterpret_cast<float*>(static_cast<char*>(workspace) + kLm2expFlagBytes)
                          : static_cast<float*>(workspace);
  const float* m_ws = b_colmax != nullptr ? b_colmax : m_buf;
  int rc = TRITURUS_B200_OK;
  // Column maxima of the result: tiles of several row tiles reduce into the array, which therefore starts
  // at -inf; a single row tile stores every column exactly once and needs no fill.
  if (out_colmax != nullptr && !plan.colmax_exclusive) {
    const int64_t n = R * K;
    const int64_t blocks = (n + 255) / 256;
    fill_neg_inf_kernel<<<static_cast<int>(blocks < 1184 ? blocks : 1184), 256, 0, st>>>(out_colmax, n);
  }
  // Every tensor map is encoded before the pre-pass is launched: the contraction kernel then follows it
  // directly in the stream, which its launch as a programmatic dependent requires.
  const bool prepass = !fused && b_colmax == nullptr;

  CUtensorMap ta, tb;
  memset(&ta, 0, sizeof(ta));
  memset(&tb, 0, sizeof(tb));
  if (gen_a) {
    // (no tensor map)
  } else if (a_mn) {
    const int64_t dims[3] = {I, J, R};
    const int64_t strides[3] = {1, as2, as0};
    const uint32_t box[3] = {32, 32, 1};
    rc = make_tmap(&ta, a, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    if (rc != TRITURUS_B200_OK) return rc;
  } else {
    const int64_t dims[3] = {J, I, R};
    const int64_t strides[3] = {1, as1, as0};
    const uint32_t box[3] = {32, 128, 1};
    rc = make_tmap(&ta, a, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TRITURUS_B200_OK) return rc;
  }
  if (gen_b) {
    // (no tensor map)
  } else if (b_km) {
    const int64_t dims[3] = {J, K, R};
    const int64_t strides[3] = {1, bs2, bs0};
    const uint32_t box[3] = {32, static_cast<uint32_t>(bn), 1};
    rc = make_tmap(&tb, b, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TRITURUS_B200_OK) return rc;
  } else {
    const int64_t dims[3] = {K, J, R};
    const int64_t strides[3] = {1, bs1, bs0};
    const uint32_t box[3] = {32, 32, 1};
    rc = make_tmap(&tb, b, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    if (rc != TRITURUS_B200_OK) return rc;
  }

  // The epilogue stores through TMA when the result meets the tensor-map rules, else with plain stores.
  CUtensorMap to;
  memset(&to, 0, sizeof(to));
  int64_t tos0 = os0, tos1 = os1;
  const bool out_tma = aligned16(out) && (K & 3) == 0 && fix_stride(I, tos1, round_up4(K)) &&
                       fix_stride(R, tos0, round_up4(K) * I);
  if (out_tma) {
    const int64_t dims[3] = {K, I, R};
    const int64_t strides[3] = {1, tos1, tos0};
    const uint32_t box[3] = {32, 32, 1};
    rc = make_tmap(&to, out, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TRITURUS_B200_OK) return rc;
  }

  Lm2expParams p;
  p.out_tma = out_tma ? 1 : 0;
  p.a_mn = a_mn ? 1 : 0;
  p.b_km = b_km ? 1 : 0;
  p.gen_a = gen_a ? 1 : 0;
  p.gen_b = gen_b ? 1 : 0;
  p.a_ptr = a;
  p.b_ptr = b;
  p.a_s0 = as_raw[0], p.a_s1 = as_raw[1], p.a_s2 = as_raw[2];
  p.b_s0 = bs_raw[0], p.b_s1 = bs_raw[1], p.b_s2 = bs_raw[2];
  p.m_ws = m_ws;
  p.out = out;
  p.out_max = out_colmax;
  p.out_s0 = os0;
  p.out_s1 = os1;
  p.R = static_cast<int>(R);
  p.I = static_cast<int>(I);
  p.J = static_cast<int>(J);
  p.K = static_cast<int>(K);
  p.tiles_m = p.tiles_n = p.num_tiles = 0;
  p.fused_max = fused ? 1 : 0;
  p.status = status_dev;

  // The TMEM-operand pair kernel takes a with j contiguous and does not fold column maxima of the result; other
  // calls run on the pair kernel that keeps the operand in shared memory.  Its b tiles are 32 rows j x 128
  // columns k, unswizzled (only the transform threads read them).
  const bool use_ts = plan.tspair && !a_mn && out_colmax == nullptr;
  CUtensorMap tb_plain;
  if (use_ts) {
    const int64_t dims[3] = {K, J, R};
    const int64_t strides[3] = {1, bs1, bs0};
    const uint32_t box[3] = {128, 32, 1};
    rc = make_tmap(&tb_plain, b, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != TRITURUS_B200_OK) return rc;
  }
  const int64_t bstr[3] = {gen_b ? bs_raw[0] : bs0, gen_b ? bs_raw[1] : bs1, gen_b ? bs_raw[2] : 1};
  if (use_ts && plan.optimistic && prepass && ws_flags) {
    // No pre-pass: the contraction takes each column's stabiliser from its first 32 rows and raises the flag
    // if a result overflowed; the exact pre-pass and contraction follow as launches that return at once
    // unless the flag is up.  Nothing clears the flag beforehand: the conditional contraction puts it down when
    // it runs, so a word that is up by accident (fresh memory) costs one exact pass and never a wrong result.
    int* flag = static_cast<int*>(workspace);
    Lm2expParams po = p;
    po.m_ws = nullptr;
    po.opt_flag = flag;
    rc = launch_lm2exp_tspair<LmTsPairOpt>(ta, tb_plain, to, po, st, false);
    if (rc != TRITURUS_B200_OK) return rc;
    // (the exact column maxima are found inside the conditional kernel: one launch behind the optimistic one)
    p.m_ws = nullptr;
    p.only_if = flag;
    p.reset_flag = flag;
    return launch_lm2exp_tspair<LmTsPairFused>(ta, tb_plain, to, p, st, true);
  }
  if (pair && !use_ts && plan.optimistic_prepass && prepass && ws_flags && out_colmax == nullptr) {
    // Pre-pass over the first 32 rows of b only; the contraction raises the flag if a result overflowed, and the
    // full pre-pass and the contraction with its maxima follow as launches that return at once unless it did.
    int* flag = static_cast<int*>(workspace);
    rc = colmax_run(b, m_buf, R, std::min<int64_t>(J, 32), K, bstr, stream, nullptr, nullptr);
    if (rc != TRITURUS_B200_OK) return rc;
    Lm2expParams po = p;
    po.opt_flag = flag;
    rc = precision == TRITURUS_B200_PRECISION_3XTF32 ? launch_lm2exp_pair<LmPairX>(ta, tb, to, po, st, true)
                                                      : launch_lm2exp_pair<LmPairT>(ta, tb, to, po, st, true);
    if (rc != TRITURUS_B200_OK) return rc;
    rc = colmax_run(b, m_buf, R, J, K, bstr, stream, flag, flag + 1);
    if (rc != TRITURUS_B200_OK) return rc;
    p.only_if = flag + 1;
    p.reset_flag = flag;
    return precision == TRITURUS_B200_PRECISION_3XTF32 ? launch_lm2exp_pair<LmPairX>(ta, tb, to, p, st, true)
                                                        : launch_lm2exp_pair<LmPairT>(ta, tb, to, p, st, true);
  }
  if (prepass && b_km) {
    for (int64_t r0 = 0; r0 < R; r0 += 65535) {  // (R <= 65535 here: one round)
      const dim3 grid(static_cast<unsigned>((K + 7) / 8), static_cast<unsigned>(std::min<int64_t>(65535, R - r0)));
      rowmax_kernel<<<grid, 256, 0, st>>>(b + r0 * bs0, m_buf + r0 * K, static_cast<int>(J), static_cast<int>(K), bs0, bs2);
    }
    if (cudaGetLastError() != cudaSuccess) return TRITURUS_B200_ELAUNCH;
  } else if (prepass) {
    rc = triturus_b200_colmax_f32(b, m_buf, R, J, K, bstr, stream);
    if (rc != TRITURUS_B200_OK) return rc;
  }
  const bool dep = prepass;
  if (use_ts) return launch_lm2exp_tspair<LmTsPair>(ta, tb_plain, to, p, st, dep);
  if (pair) {
    return precision == TRITURUS_B200_PRECISION_3XTF32 ? launch_lm2exp_pair<LmPairX>(ta, tb, to, p, st, dep)
                                                        : launch_lm2exp_pair<LmPairT>(ta, tb, to, p, st, dep);
  }
  auto single = [&](const Lm2expParams& q, bool dependent) -> int {
    if (b_km || gen_a || gen_b) {
      if (precision == TRITURUS_B200_PRECISION_3XTF32) {
        return mt == 2 ? launch_lm2exp<LmXo_128_2>(ta, tb, to, q, st, dependent)
                       : launch_lm2exp<LmXo_128_1>(ta, tb, to, q, st, dependent);
      }
      if (bn == 256)
        return mt == 2 ? launch_lm2exp<LmTo_256_2>(ta, tb, to, q, st, dependent)
                       : launch_lm2exp<LmTo_256_1>(ta, tb, to, q, st, dependent);
      if (plan.promote_tf32)
        return mt == 2 ? launch_lm2exp<LmPo_128_2>(ta, tb, to, q, st, dependent)
                       : launch_lm2exp<LmPo_128_1>(ta, tb, to, q, st, dependent);
      return mt == 2 ? launch_lm2exp<LmTo_128_2>(ta, tb, to, q, st, dependent)
                     : launch_lm2exp<LmTo_128_1>(ta, tb, to, q, st, dependent);
    }
    if (precision == TRITURUS_B200_PRECISION_3XTF32) {
      return mt == 2 ? launch_lm2exp<LmX_128_2>(ta, tb, to, q, st, dependent)
                     : launch_lm2exp<LmX_128_1>(ta, tb, to, q, st, dependent);
    }
    if (bn == 256)
      return mt == 2 ? launch_lm2exp<LmT_256_2>(ta, tb, to, q, st, dependent)
                     : launch_lm2exp<LmT_256_1>(ta, tb, to, q, st, dependent);
    if (plan.promote_tf32)
      return mt == 2 ? launch_lm2exp<LmP_128_2>(ta, tb, to, q, st, dependent)
                     : launch_lm2exp<LmP_128_1>(ta, tb, to, q, st, dependent);
    return mt == 2 ? launch_lm2exp<LmT_128_2>(ta, tb, to, q, st, dependent)
                   : launch_lm2exp<LmT_128_1>(ta, tb, to, q, st, dependent);
  };
  if (fused && plan.optimistic_fused && ws_flags && out_colmax == nullptr) {
    // The max pass scans only the first k-block of each slab; a launch that saw a result overflow raises the
    // flag, and the same kernel with the full max pass follows as a launch that returns at once unless the flag
    // is up (its last CTA then puts it down again).
    int* flag = static_cast<int*>(workspace);
    Lm2expParams po = p;
    po.opt_flag = flag;
    rc = single(po, false);
    if (rc != TRITURUS_B200_OK) return rc;
    p.only_if = flag;
    p.reset_flag = flag;
    return single(p, true);
  }
  return single(p, dep);
}

// Batches of more than 65535 entries (the limit of gridDim.y / .z in the small kernels) run block by block on
// the same stream; the reference's 1-D grid takes any batch (triturus/lm2exp.py:177-181).
constexpr int64_t kMaxBatchBlock = 65535;

static int lm2exp_run(const float* a, const float* b, float* out, int64_t R, int64_t I, int64_t J, int64_t K,
                      const int64_t a_strides[3], const int64_t b_strides[3], const int64_t out_strides[3],
                      int precision, int variant, const float* b_colmax, float* out_colmax, void* workspace,
                      size_t workspace_bytes, int32_t* status_dev, void* stream) {
  if (R <= kMaxBatchBlock || a == nullptr || b == nullptr || out == nullptr || a_strides == nullptr ||
      b_strides == nullptr || out_strides == nullptr)
    return lm2exp_run_block(a, b, out, R, I, J, K, a_strides, b_strides, out_strides, precision, variant, b_colmax,
                            out_colmax, workspace, workspace_bytes, status_dev, stream);
  for (int64_t r0 = 0; r0 < R; r0 += kMaxBatchBlock) {
    const int64_t n = std::min(kMaxBatchBlock, R - r0);
    const int rc = lm2exp_run_block(a + r0 * a_strides[0], b + r0 * b_strides[0], out + r0 * out_strides[0], n, I, J,
                                    K, a_strides, b_strides, out_strides, precision, variant,
                                    b_colmax != nullptr ? b_colmax + r0 * K : nullptr,
                                    out_colmax != nullptr ? out_colmax + r0 * K : nullptr, workspace, workspace_bytes,
                                    status_dev, stream);
    if (rc != TRITURUS_B200_OK) return rc;
  }
  return TRITURUS_B200_OK;
}

int triturus_b200_mm_f32(const float* a, const float* b, float* out, int64_t M, int64_t K, int64_t N,
                         const int64_t a_strides[2], const int64_t b_strides[2], const int64_t out_strides[2],
                         int precision, int32_t* status_dev, void* stream) {
  if (a == nullptr || b == nullptr || out == nullptr || a_strides == nullptr || b_strides == nullptr ||
      out_strides == nullptr)
    return TRITURUS_B200_EINVAL;
  if (M <= 0 || K <= 0 || N <= 0 || M > (1 << 30) || K > (1 << 30) || N > (1 << 30)) return TRITURUS_B200_EINVAL;
  if (precision != TRITURUS_B200_PRECISION_TF32 && precision != TRITURUS_B200_PRECISION_3XTF32)
    return TRITURUS_B200_EINVAL;
  // out[i, k] = sum_j a[i, j] * b[j, k]: the lm2exp pipeline on one batch entry with the transform switched off
  int64_t as0 = a_strides[0], bs0 = b_strides[0], os0 = out_strides[0];
  if ((K > 1 && a_strides[1] != 1) || (N > 1 && (b_strides[1] != 1 || out_strides[1] != 1))) return TRITURUS_B200_EALIGN;
  if (!aligned16(a) || !aligned16(b)) return TRITURUS_B200_EALIGN;
  if (!fix_stride(M, as0, round_up4(K)) || !fix_stride(K, bs0, round_up4(N))) return TRITURUS_B200_EALIGN;
  if (M > 1 && os0 <= 0) return TRITURUS_B200_EALIGN;
  CUtensorMap ta, tb, to;
  memset(&to, 0, sizeof(to));
  int rc;
  {
    const int64_t dims[3] = {K, M, 1};
    const int64_t strides[3] = {1, as0, as0 * M};
    const uint32_t box[3] = {32, 128, 1};
    rc = make_tmap(&ta, a, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TRITURUS_B200_OK) return rc;
  }
  {
    const int64_t dims[3] = {N, K, 1};
    const int64_t strides[3] = {1, bs0, bs0 * K};
    const uint32_t box[3] = {32, 32, 1};
    rc = make_tmap(&tb, b, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    if (rc != TRITURUS_B200_OK) return rc;
  }
  int64_t tos0 = os0;
  const bool out_tma = aligned16(out) && (N & 3) == 0 && fix_stride(M, tos0, round_up4(N));
  if (out_tma) {
    const int64_t dims[3] = {N, M, 1};
    const int64_t strides[3] = {1, tos0, tos0 * M};
    const uint32_t box[3] = {32, 32, 1};
    rc = make_tmap(&to, out, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TRITURUS_B200_OK) return rc;
  }
  Lm2expParams p;
  p.out_tma = out_tma ? 1 : 0;
  p.a_mn = 0;
  p.m_ws = nullptr;
  p.out = out;
  p.out_max = nullptr;
  p.out_s0 = os0 * M;
  p.out_s1 = os0;
  p.R = 1;
  p.I = static_cast<int>(M);
  p.J = static_cast<int>(K);
  p.K = static_cast<int>(N);
  p.tiles_m = p.tiles_n = p.num_tiles = 0;
  p.fused_max = 0;
  p.status = status_dev;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return precision == TRITURUS_B200_PRECISION_3XTF32 ? launch_lm2exp<LmPlainX>(ta, tb, to, p, st, false)
                                                      : launch_lm2exp<LmPlainT>(ta, tb, to, p, st, false);
}

int triturus_b200_lm2exp_f32(const float* a, const float* b, float* out, int64_t R, int64_t I, int64_t J, int64_t K,
                             const int64_t a_strides[3], const int64_t b_strides[3], const int64_t out_strides[3],
                             int precision, int variant, void* workspace, size_t workspace_bytes,
                             int32_t* status_dev, void* stream) {
  return lm2exp_run(a, b, out, R, I, J, K, a_strides, b_strides, out_strides, precision, variant, nullptr, nullptr,
                    workspace, workspace_bytes, status_dev, stream);
}

int triturus_b200_lm2exp_chain_f32(const float* a, const float* b, float* out, int64_t R, int64_t I, int64_t J,
                                   int64_t K, const int64_t a_strides[3], const int64_t b_strides[3],
                                   const int64_t out_strides[3], int precision, int variant, const float* b_colmax,
                                   float* out_colmax, void* workspace, size_t workspace_bytes, int32_t* status_dev,
                                   void* stream) {
  return lm2exp_run(a, b, out, R, I, J, K, a_strides, b_strides, out_strides, precision, variant, b_colmax,
                    out_colmax, workspace, workspace_bytes, status_dev, stream);
}

int triturus_b200_lm2exp_chain_launches(int64_t R, int64_t I, int64_t J, int64_t K, int precision, int variant,
                                        int have_b_colmax, int want_out_colmax) {
  if (R <= 0 || I <= 0 || J <= 0 || K <= 0) return TRITURUS_B200_EINVAL;
  if (precision != TRITURUS_B200_PRECISION_TF32 && precision != TRITURUS_B200_PRECISION_3XTF32)
    return TRITURUS_B200_EINVAL;
  Lm2expPlan plan;
  const int rc = plan_lm2exp(R, I, J, K, precision, variant, &plan, have_b_colmax != 0);
  if (rc != TRITURUS_B200_OK) return rc;
  if ((plan.optimistic || plan.optimistic_fused) && !want_out_colmax) return 2;  // as triturus_b200_lm2exp_launches
  if (plan.optimistic_prepass && !want_out_colmax) return 4;
  return 1 + ((plan.fused || have_b_colmax) ? 0 : 1) + ((want_out_colmax && !plan.colmax_exclusive) ? 1 : 0);
}

}  // extern "C"

// ----------------------------------------------------------------------------- lt2exp launch

namespace tb200 {

// How the contraction of a launch is shared out (see LtWork in lt2exp_kernel.cuh).
struct LtSplit {
  int nsplit;  // equal slices per tile, one work item each (1: whole tiles)
  int stream;  // 1: every CTA gets the same number of k-blocks of the whole launch, across tile borders
};

// request: 0 = automatic, 1 = never split (deterministic), 9999 = automatic but split in any case,
// 9998 = stream, anything else = that many slices per tile.
//  * Few tiles (they would occupy at most half the SMs): slices, enough to cover the SMs, each at least
//    kMinSliceBlocks k-blocks long so the pipeline fill and the per-item column maxima stay a small part.
//  * A last wave that is less than 90 % full on a contraction of at least kMinStreamBlocks k-blocks per tile:
//    stream, which keeps every SM busy to the end (R = 8 entries of 256 x 4096 results on 256 x 256 tiles are
//    128 tiles on 148 SMs: 0.86 of a wave).  A CTA then works on up to two partial tiles besides its whole
//    ones (prologue and epilogue of each cost about as much as 50 k-blocks), hence the minimum length.
// auto_stream: the launch can complete shared tiles through scratch memory (see Lt2expParams::park); without
// it the end-to-end form would have to add every partial sum into the result with atomics, which costs more
// than the ragged wave it removes, so the automatic choice then keeps whole tiles.
static LtSplit lt2exp_split(int64_t tiles, int I, int J, int request, bool auto_stream) {
  constexpr int kMinSliceBlocks = 16;
  constexpr int kMinStreamBlocks = 256;
  const int JC = (J + 31) / 32;
  const int64_t kb = static_cast<int64_t>(JC) * I;
  const int sms = sm_count();
  LtSplit sp{1, 0};
  if (request == 1) return sp;
  if (request == 9998) {
    sp.stream = 1;
    return sp;
  }
  int64_t want = request;
  if (request == 0 || request == 9999) {
    want = tiles * 2 > sms ? 1 : sms / tiles;
    // Two more launches (zero-fill and log pass) cost about as much as 50 k-blocks of the main loop: a
    // contraction shorter than that is left whole.
    if (request == 0 && kb < 64) want = 1;
    if (request == 9999 && want < 2) want = 2;
    if (want == 1 && tiles > sms / 2) {
      const int64_t waves = (tiles + sms - 1) / sms;
      const bool ragged = tiles * 10 < waves * sms * 9;  // last wave under 90 % full
      if (auto_stream && ragged && kb >= kMinStreamBlocks && waves <= 8) sp.stream = 1;
      return sp;
    }
  }
  if (want > kb / kMinSliceBlocks) want = kb / kMinSliceBlocks;
  if (want < 1) want = 1;
  sp.nsplit = static_cast<int>(want);
  return sp;
}

// What a launch function is asked to do: launch, or (query != nullptr) only report what it would launch.
struct LtQuery {
  int launches;     // kernels per call
  int split_code;   // 1 = whole tiles, n = slices per tile, 9998 = end to end
  size_t ws_bytes;  // scratch memory the plan uses (0: none)
};
struct LtLaunch {
  int split_request;
  cudaStream_t stream;
  LtQuery* query;   // queries assume that the caller will supply the scratch memory they report
  void* ws;         // scratch memory of the call (may be null)
  size_t ws_bytes;
};

constexpr size_t kParkHeader = 1024;  // flags (one int per CTA) ahead of the parked tiles

template <class Cfg, void (*Kern)(const CUtensorMap, const Lt2expParams), bool CAN_PARK>
static int launch_lt2exp_with(const CUtensorMap& tw, Lt2expParams p, const LtLaunch& L) {
  auto kern = Kern;
  static std::once_flag once[64];
  static cudaError_t attr_rc[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return TRITURUS_B200_ELAUNCH;
  p.tiles_m = (p.S + Cfg::BM * Cfg::MT - 1) / (Cfg::BM * Cfg::MT);
  p.tiles_n = (p.K + Cfg::BN - 1) / Cfg::BN;
  const int64_t nt = static_cast<int64_t>(p.R) * p.tiles_m * p.tiles_n;
  if (nt > INT32_MAX) return TRITURUS_B200_EINVAL;
  p.num_tiles = static_cast<int>(nt);
  // Scratch memory for the end-to-end form: one parked tile per CTA behind the flags.
  const size_t park_need = kParkHeader + static_cast<size_t>(sm_count()) * Cfg::MT * Cfg::BM * Cfg::BN * sizeof(float);
  const bool have_ws = CAN_PARK && sm_count() * sizeof(int) <= kParkHeader &&
                       (L.query != nullptr || (L.ws != nullptr && L.ws_bytes >= park_need &&
                                               (reinterpret_cast<uintptr_t>(L.ws) & 255) == 0));
  // Not chosen automatically for a launch that re-sums its accumulator in chunks (3xTF32, long plain-TF32
  // contractions): sharing tiles made those slower (R32 256^4: 1.32 against 0.81 ms in TF32, 2.87 against 1.68 ms
  // in 3xTF32; R128: 2.75 against 2.40 ms), the explicit request 9998 still selects it.
  const bool chunked = Cfg::PROMOTE && static_cast<int64_t>((p.J + 31) / 32) * p.I > Cfg::CHUNK;
  const LtSplit sp = lt2exp_split(nt, p.I, p.J, L.split_request, have_ws && !chunked);
  p.nsplit = sp.nsplit;
  p.stream = sp.stream;
  const int64_t items = nt * sp.nsplit;
  if (items > INT32_MAX) return TRITURUS_B200_EINVAL;
  p.num_items = static_cast<int>(items);
  if (sp.stream) {
    // Whole waves first, then the tiles of the last wave shared among all CTAs (LtWork in lt2exp_kernel.cuh).
    const int G = sm_count();
    const int64_t kbt = static_cast<int64_t>((p.J + 31) / 32) * p.I;
    const int64_t waves = (nt + G - 1) / G;
    p.lw_first = static_cast<int>((waves - 1) * G);
    const int rem = static_cast<int>(nt - p.lw_first);
    p.lw_parts = 1;
    p.lw_main = static_cast<int>(kbt);
    if (rem * 2 <= G) {
      int64_t parts = G / rem;
      if (parts > 8) parts = 8;  // shorter parts are mostly prologue and epilogue
      if (parts > kbt) parts = kbt;
      p.lw_parts = static_cast<int>(parts < 1 ? 1 : parts);
    } else if (rem < G && kbt >= 2) {
      // mains and tails: a CTA with the most tails (q of them) is busy as long as a main part, counting for
      // every work item a prologue and epilogue worth kItemBlocks k-blocks (measured: 25 us per tail of a
      // 256 x 256 tile against 0.73 us per k-block): q * (kbt - x + o) = x + o
      constexpr int64_t kItemBlocks = 32;
      const int h = G - rem;
      const int64_t q = (rem + h - 1) / h;
      int64_t x = ((q * (kbt + kItemBlocks) - kItemBlocks) / (q + 1)) & ~int64_t(7);
      if (x < 1) x = 1;
      if (x > kbt - 1) x = kbt - 1;
      p.lw_parts = 0;
      p.lw_main = static_cast<int>(x);
    }
  } else {
    p.lw_first = p.num_tiles;
    p.lw_parts = 1;
    p.lw_main = 0;
  }
  const bool parked = sp.stream != 0 && have_ws;             // shared tiles completed through the scratch memory
  const bool split = (sp.nsplit > 1 || sp.stream != 0) && !parked;  // ... or with additions into the zero-filled result
  // the log pass of a split launch runs on a (K / 128, S / 64, R) grid
  if (split && (p.S + 63) / 64 > 65535) return TRITURUS_B200_EINVAL;
  if (L.query != nullptr) {
    L.query->launches = split ? 3 : 1;
    L.query->split_code = sp.stream ? 9998 : sp.nsplit;
    L.query->ws_bytes = parked ? park_need : 0;
    return TRITURUS_B200_OK;
  }
  std::call_once(once[dev], [&] {
    attr_rc[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  });
  if (attr_rc[dev] != cudaSuccess) return TRITURUS_B200_ELAUNCH;
  p.park = nullptr;
  p.park_flags = nullptr;
  if (parked) {
    p.park_flags = static_cast<int*>(L.ws);
    p.park = reinterpret_cast<float*>(static_cast<uint8_t*>(L.ws) + kParkHeader);
    if (cudaMemsetAsync(L.ws, 0, kParkHeader, L.stream) != cudaSuccess) return TRITURUS_B200_ELAUNCH;
  }
  if (split) {
    const int64_t total = static_cast<int64_t>(p.R) * p.S * p.K;
    const int64_t zb = (total + 255) / 256;
    lt2exp_zero_kernel<<<static_cast<int>(zb < 4 * sm_count() ? zb : 4 * sm_count()), 256, 0, L.stream>>>(
        p.out, p.out_s0, p.out_s1, p.R, p.S, p.K);
  }
  const int grid = (sp.stream || p.num_items >= sm_count()) ? sm_count() : p.num_items;
  kern<<<grid, Cfg::NTHREADS, Cfg::SMEM_BYTES, L.stream>>>(tw, p);
  if (split) {
    const dim3 fgrid((p.K + 127) / 128, (p.S + 63) / 64, p.R);
    if (Cfg::PREC) lt2exp_finish_kernel<1><<<fgrid, 256, 0, L.stream>>>(p);
    else lt2exp_finish_kernel<0><<<fgrid, 256, 0, L.stream>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? TRITURUS_B200_OK : TRITURUS_B200_ELAUNCH;
}

template <class Cfg>
static int launch_lt2exp(const CUtensorMap& tw, Lt2expParams p, const LtLaunch& L) {
  return launch_lt2exp_with<Cfg, lt2exp_kernel<Cfg>, true>(tw, p, L);
}

// (the kernels that keep the generated operand in tensor memory complete shared tiles with additions only)
template <class Cfg>
static int launch_lt2exp_tmem(const CUtensorMap& tw, Lt2expParams p, const LtLaunch& L) {
  return launch_lt2exp_with<Cfg, lt2exp_tmem_kernel<Cfg>, false>(tw, p, L);
}

//                              MT NS   (generated operand in TMEM, 128 columns k per tile, TF32)
using LtM_1 = Lt2expTmemCfg<1, 8>;
using LtM_2 = Lt2expTmemCfg<2, 6>;
using LtM_1x2 = Lt2expTmemCfg<1, 4, 2>;  // 128 rows x two 128-column blocks sharing each w tile

//                          BN   MT PREC NS NTW
using LtT_128_1 = Lt2expCfg<128, 1, 0, 6, 8>;
using LtT_128_2 = Lt2expCfg<128, 2, 0, 4, 8>;
using LtT_256_1 = Lt2expCfg<256, 1, 0, 4, 8>;
using LtT_256_2 = Lt2expCfg<256, 2, 0, 3, 8>;
using LtX_128_1 = Lt2expCfg<128, 1, 1, 3, 8>;
using LtX_128_2 = Lt2expCfg<128, 2, 1, 2, 8>;
using LtX_256_1 = Lt2expCfg<256, 1, 1, 2, 8>;
// plain TF32 with chunked re-summation of the accumulator (contractions of more than 32 K terms)
using LtP_128_1 = Lt2expCfg<128, 1, 0, 6, 8, true>;
using LtP_128_2 = Lt2expCfg<128, 2, 0, 4, 8, true>;
using LtP_256_1 = Lt2expCfg<256, 1, 0, 4, 8, true>;

}  // namespace tb200

// Decodes SPLIT * 10000 + BN * 10 + MT, filling in the automatic tile shape.
// *promote: plain TF32 over a contraction of more than kLongContraction terms on a tile whose accumulator
// leaves room for a master copy in TMEM (the automatic choice is restricted to such tiles; an explicit
// 256 x 256 tile or TMEM-operand variant is honoured and runs without the re-summation).
static int lt2exp_variant(int variant, int precision, int64_t R, int64_t S, int64_t I, int64_t J, int64_t K, int* bn,
                          int* mt, int* split, bool* promote) {
  if (variant < 0) return TRITURUS_B200_EINVAL;
  *split = variant / 10000;
  int tile = variant % 10000;
  const bool long_tf = precision == TRITURUS_B200_PRECISION_TF32 && I * ((J + 31) / 32 * 32) > tb200::kLongContraction;
  if (tile == 0) {
    tile = tb200::auto_variant(R, S, K, true, false, long_tf ? 256 : 512);
    // 128 rows x 256 columns in TF32: the kernel that keeps the generated operand in TMEM moves a third of
    // the shared-memory bytes per k-block (measured 8 % faster on such tiles).
    if (tile == 2561 && precision == TRITURUS_B200_PRECISION_TF32 && !long_tf) tile = 1285;
  }
  *bn = tile / 10;
  *mt = tile % 10;
  // 3xTF32 keeps hi and lo copies of both operands: two row blocks leave room for 128 columns only
  if (precision == TRITURUS_B200_PRECISION_3XTF32 && *bn == 256 && *mt == 2) *bn = 128;
  *promote = long_tf && (tile == 1281 || tile == 1282 || tile == 2561);
  // operand in TMEM: 128 columns x 128 / 256 rows (1283 / 1284), 256 columns x 128 rows (1285)
  if (*bn == 128 && (*mt == 3 || *mt == 4 || *mt == 5)) return TRITURUS_B200_OK;
  if ((*bn != 128 && *bn != 256) || (*mt != 1 && *mt != 2)) return TRITURUS_B200_EINVAL;
  return TRITURUS_B200_OK;
}

static int lt2exp_check_dims(int64_t R, int64_t S, int64_t I, int64_t J, int64_t K, int precision) {
  if (R <= 0 || S <= 0 || I <= 0 || J <= 0 || K <= 0) return TRITURUS_B200_EINVAL;
  if (R > INT32_MAX || S > (1 << 30) || I > (1 << 24) || J > (1 << 24) || K > (1 << 30)) return TRITURUS_B200_EINVAL;
  if (((J + 31) / 32) * I > (1 << 28)) return TRITURUS_B200_EINVAL;
  if (precision != TRITURUS_B200_PRECISION_TF32 && precision != TRITURUS_B200_PRECISION_3XTF32)
    return TRITURUS_B200_EINVAL;
  return TRITURUS_B200_OK;
}

template <class... Args>
static int lt2exp_dispatch(int precision, int bn, int mt, bool promote, Args... args) {
  using namespace tb200;
  if (promote) {
    if (bn == 256) return launch_lt2exp<LtP_256_1>(args...);
    return mt == 2 ? launch_lt2exp<LtP_128_2>(args...) : launch_lt2exp<LtP_128_1>(args...);
  }
  if (mt == 3 || mt == 4 || mt == 5) {
    if (precision != TRITURUS_B200_PRECISION_TF32) return TRITURUS_B200_EINVAL;
    if (mt == 5) return launch_lt2exp_tmem<LtM_1x2>(args...);
    return mt == 4 ? launch_lt2exp_tmem<LtM_2>(args...) : launch_lt2exp_tmem<LtM_1>(args...);
  }
  if (precision == TRITURUS_B200_PRECISION_3XTF32) {
    if (bn == 256 && mt == 1) return launch_lt2exp<LtX_256_1>(args...);
    return mt == 2 ? launch_lt2exp<LtX_128_2>(args...) : launch_lt2exp<LtX_128_1>(args...);
  }
  if (bn == 256) return mt == 2 ? launch_lt2exp<LtT_256_2>(args...) : launch_lt2exp<LtT_256_1>(args...);
  return mt == 2 ? launch_lt2exp<LtT_128_2>(args...) : launch_lt2exp<LtT_128_1>(args...);
}

static int lt2exp_query(int64_t R, int64_t S, int64_t I, int64_t J, int64_t K, int precision, int variant,
                        tb200::LtQuery* q, int* tile_code) {
  int rc = lt2exp_check_dims(R, S, I, J, K, precision);
  if (rc != TRITURUS_B200_OK) return rc;
  int bn, mt, split;
  bool promote;
  rc = lt2exp_variant(variant, precision, R, S, I, J, K, &bn, &mt, &split, &promote);
  if (rc != TRITURUS_B200_OK) return rc;
  tb200::Lt2expParams p{};
  p.R = static_cast<int>(R);
  p.S = static_cast<int>(S);
  p.I = static_cast<int>(I);
  p.J = static_cast<int>(J);
  p.K = static_cast<int>(K);
  CUtensorMap none{};
  const tb200::LtLaunch L{split, static_cast<cudaStream_t>(nullptr), q, nullptr, 0};
  rc = lt2exp_dispatch(precision, bn, mt, promote, none, p, L);
  *tile_code = bn * 10 + mt;
  return rc;
}

extern "C" int triturus_b200_lt2exp_launches(int64_t R, int64_t S, int64_t I, int64_t J, int64_t K, int precision,
                                             int variant) {
  tb200::LtQuery q{};
  int tile = 0;
  const int rc = lt2exp_query(R, S, I, J, K, precision, variant, &q, &tile);
  return rc == TRITURUS_B200_OK ? q.launches : rc;
}

extern "C" int triturus_b200_lt2exp_plan(int64_t R, int64_t S, int64_t I, int64_t J, int64_t K, int precision,
                                         int variant) {
  tb200::LtQuery q{};
  int tile = 0;
  const int rc = lt2exp_query(R, S, I, J, K, precision, variant, &q, &tile);
  return rc == TRITURUS_B200_OK ? q.split_code * 10000 + tile : rc;
}

extern "C" size_t triturus_b200_lt2exp_workspace_bytes(int64_t R, int64_t S, int64_t I, int64_t J, int64_t K,
                                                       int precision, int variant) {
  tb200::LtQuery q{};
  int tile = 0;
  const int rc = lt2exp_query(R, S, I, J, K, precision, variant, &q, &tile);
  return rc == TRITURUS_B200_OK ? q.ws_bytes : 0;
}

// Shared body of the lt2exp entry points.  a_colmax / b_colmax (optional, both or neither): [R, K] column
// maxima of a and b, which replace the scan at the start of every tile.  out_colmax (optional): [R, K] receives
// max_s out[r, s, k].
static int lt2exp_run_block(const float* w, const float* a, const float* b, float* out, int64_t R, int64_t S, int64_t I,
                      int64_t J, int64_t K, const int64_t w_strides[4], const int64_t a_strides[3],
                      const int64_t b_strides[3], const int64_t out_strides[3], int precision, int variant,
                      const float* a_colmax, const float* b_colmax, float* out_colmax, void* workspace,
                      size_t workspace_bytes, int32_t* status_dev, void* stream) {
  if ((a_colmax == nullptr) != (b_colmax == nullptr)) return TRITURUS_B200_EINVAL;
  if (out_colmax != nullptr && (out_colmax == a_colmax || out_colmax == b_colmax)) return TRITURUS_B200_EINVAL;
  if (w == nullptr || a == nullptr || b == nullptr || out == nullptr || w_strides == nullptr ||
      a_strides == nullptr || b_strides == nullptr || out_strides == nullptr)
    return TRITURUS_B200_EINVAL;
  {
    const int rc = lt2exp_check_dims(R, S, I, J, K, precision);
    if (rc != TRITURUS_B200_OK) return rc;
  }

  int64_t ws0 = w_strides[0], ws1 = w_strides[1], ws2 = w_strides[2], ws3 = w_strides[3];
  int64_t as0 = a_strides[0], as1 = a_strides[1], as2 = a_strides[2];
  int64_t bs0 = b_strides[0], bs1 = b_strides[1], bs2 = b_strides[2];
  int64_t os0 = out_strides[0], os1 = out_strides[1], os2 = out_strides[2];
  // w goes through a tensor map; a and b are read with ordinary loads, 4 bytes at a time unless vec_ab holds, and
  // may have any strides (the reference forwards whatever it is given, triturus/lt2exp.py:580-585 and :612-617).
  if ((J > 1 && ws3 != 1) || (K > 1 && os2 != 1)) return TRITURUS_B200_EALIGN;
  if (!aligned16(w) || (reinterpret_cast<uintptr_t>(a) & 3) != 0 || (reinterpret_cast<uintptr_t>(b) & 3) != 0)
    return TRITURUS_B200_EALIGN;
  if (K == 1) as2 = bs2 = 1;
  const int64_t j4 = round_up4(J);
  if (!fix_stride(I, ws2, j4) || !fix_stride(S, ws1, j4 * I) || !fix_stride(R, ws0, j4 * I * S))
    return TRITURUS_B200_EALIGN;
  if ((S > 1 && os1 <= 0) || (R > 1 && os0 <= 0)) return TRITURUS_B200_EALIGN;

  int bn, mt, split;
  bool promote;
  {
    const int rc = lt2exp_variant(variant, precision, R, S, I, J, K, &bn, &mt, &split, &promote);
    if (rc != TRITURUS_B200_OK) return rc;
  }

  CUtensorMap tw;
  {
    const int64_t dims[4] = {J, I, S, R};
    const int64_t strides[4] = {1, ws2, ws1, ws0};
    const uint32_t box[4] = {32, 1, 128, 1};
    const int rc = make_tmap(&tw, w, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TRITURUS_B200_OK) return rc;
  }

  Lt2expParams p;
  p.a = a;
  p.b = b;
  p.out = out;
  p.a_s0 = as0;
  p.a_s1 = as1;
  p.b_s0 = bs0;
  p.b_s1 = bs1;
  p.a_s2 = as2;
  p.b_s2 = bs2;
  p.out_s0 = os0;
  p.out_s1 = os1;
  p.R = static_cast<int>(R);
  p.S = static_cast<int>(S);
  p.I = static_cast<int>(I);
  p.J = static_cast<int>(J);
  p.K = static_cast<int>(K);
  p.tiles_m = p.tiles_n = p.num_tiles = 0;
  p.vec_ab = (K % 4 == 0 && as2 == 1 && bs2 == 1 && aligned16(a) && aligned16(b) && as0 % 4 == 0 && as1 % 4 == 0 &&
              bs0 % 4 == 0 && bs1 % 4 == 0) ? 1 : 0;
  p.status = status_dev;
  p.ma_in = a_colmax;
  p.mb_in = b_colmax;
  p.out_max = out_colmax;
  if (out_colmax != nullptr) {
    const int64_t n = R * K;
    const int64_t blocks = (n + 255) / 256;
    tb200::fill_neg_inf_kernel<<<static_cast<int>(blocks < 1184 ? blocks : 1184), 256, 0,
                                 static_cast<cudaStream_t>(stream)>>>(out_colmax, n);
  }

  const tb200::LtLaunch L{split, static_cast<cudaStream_t>(stream), nullptr, workspace, workspace_bytes};
  return lt2exp_dispatch(precision, bn, mt, promote, tw, p, L);
}

static int lt2exp_run(const float* w, const float* a, const float* b, float* out, int64_t R, int64_t S, int64_t I,
                      int64_t J, int64_t K, const int64_t w_strides[4], const int64_t a_strides[3],
                      const int64_t b_strides[3], const int64_t out_strides[3], int precision, int variant,
                      const float* a_colmax, const float* b_colmax, float* out_colmax, void* workspace,
                      size_t workspace_bytes, int32_t* status_dev, void* stream) {
  if (R <= kMaxBatchBlock || w == nullptr || a == nullptr || b == nullptr || out == nullptr ||
      w_strides == nullptr || a_strides == nullptr || b_strides == nullptr || out_strides == nullptr)
    return lt2exp_run_block(w, a, b, out, R, S, I, J, K, w_strides, a_strides, b_strides, out_strides, precision,
                            variant, a_colmax, b_colmax, out_colmax, workspace, workspace_bytes, status_dev, stream);
  for (int64_t r0 = 0; r0 < R; r0 += kMaxBatchBlock) {
    const int64_t n = std::min(kMaxBatchBlock, R - r0);
    const int rc = lt2exp_run_block(w + r0 * w_strides[0], a + r0 * a_strides[0], b + r0 * b_strides[0],
                                    out + r0 * out_strides[0], n, S, I, J, K, w_strides, a_strides, b_strides,
                                    out_strides, precision, variant, a_colmax != nullptr ? a_colmax + r0 * K : nullptr,
                                    b_colmax != nullptr ? b_colmax + r0 * K : nullptr,
                                    out_colmax != nullptr ? out_colmax + r0 * K : nullptr, workspace, workspace_bytes,
                                    status_dev, stream);
    if (rc != TRITURUS_B200_OK) return rc;
  }
  return TRITURUS_B200_OK;
}

extern "C" int triturus_b200_lt2exp_f32(const float* w, const float* a, const float* b, float* out, int64_t R,
                                        int64_t S, int64_t I, int64_t J, int64_t K, const int64_t w_strides[4],
                                        const int64_t a_strides[3], const int64_t b_strides[3],
                                        const int64_t out_strides[3], int precision, int variant,
                                        int32_t* status_dev, void* stream) {
  return lt2exp_run(w, a, b, out, R, S, I, J, K, w_strides, a_strides, b_strides, out_strides, precision, variant,
                    nullptr, nullptr, nullptr, nullptr, 0, status_dev, stream);
}

extern "C" int triturus_b200_lt2exp_ws_f32(const float* w, const float* a, const float* b, float* out, int64_t R,
                                           int64_t S, int64_t I, int64_t J, int64_t K, const int64_t w_strides[4],
                                           const int64_t a_strides[3], const int64_t b_strides[3],
                                           const int64_t out_strides[3], int precision, int variant, void* workspace,
                                           size_t workspace_bytes, int32_t* status_dev, void* stream) {
  return lt2exp_run(w, a, b, out, R, S, I, J, K, w_strides, a_strides, b_strides, out_strides, precision, variant,
                    nullptr, nullptr, nullptr, workspace, workspace_bytes, status_dev, stream);
}

extern "C" int triturus_b200_lt2exp_chain_f32(const float* w, const float* a, const float* b, float* out, int64_t R,
                                              int64_t S, int64_t I, int64_t J, int64_t K,
                                              const int64_t w_strides[4], const int64_t a_strides[3],
                                              const int64_t b_strides[3], const int64_t out_strides[3],
                                              int precision, int variant, const float* a_colmax,
                                              const float* b_colmax, float* out_colmax, int32_t* status_dev,
                                              void* stream) {
  return lt2exp_run(w, a, b, out, R, S, I, J, K, w_strides, a_strides, b_strides, out_strides, precision, variant,
                    a_colmax, b_colmax, out_colmax, nullptr, 0, status_dev, stream);
}

// ----------------------------------------------------------------------------- lm2exp without caller scratch
//
// Some callers of this library are not allowed to allocate device memory at the point where they call
// it: code running inside a memory-pool or arena that owns all of HBM, real-time loops that forbid
// cudaMalloc because it synchronises the device, and plugin hosts that hand out only input and output
// buffers.  For them the stabiliser scratch lives in the library image itself.
//
// The array below is device memory reserved at module load on every GPU that loads this library
// (4 MiB per GPU, held until the process exits).  Its name is only meaningful to device code; host code
// must not pass it to a kernel as if it were a pointer.  The host obtains the real device address once
// per device with cudaGetSymbolAddress and passes that.

#define TRITURUS_B200_STATIC_STAB_FLOATS (1 << 20)

static __device__ __align__(256) float g_static_stab[TRITURUS_B200_STATIC_STAB_FLOATS];

namespace tb200 {

// Device address of g_static_stab on the current device, resolved on first use per device.
static int static_stab_address(float** out) {
  static float* addr[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TRITURUS_B200_ELAUNCH;
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_stab) != cudaSuccess || p == nullptr) return TRITURUS_B200_ELAUNCH;
    addr[dev] = static_cast<float*>(p);
  }
  *out = addr[dev];
  return TRITURUS_B200_OK;
}

}  // namespace tb200

extern "C" size_t triturus_b200_lm2exp_static_max_columns(void) { return TRITURUS_B200_STATIC_STAB_FLOATS; }

extern "C" int triturus_b200_lm2exp_f32_static(const float* a, const float* b, float* out, int64_t R, int64_t I,
                                               int64_t J, int64_t K, const int64_t a_strides[3],
                                               const int64_t b_strides[3], const int64_t out_strides[3],
                                               int precision, int variant, int32_t* status_dev, void* stream) {
  if (R <= 0 || K <= 0) return TRITURUS_B200_EINVAL;
  // R * K stabiliser values must fit the built-in array; larger problems need the entry point that takes
  // a caller workspace.
  if (R > TRITURUS_B200_STATIC_STAB_FLOATS || K > TRITURUS_B200_STATIC_STAB_FLOATS ||
      R * K > TRITURUS_B200_STATIC_STAB_FLOATS)
    return TRITURUS_B200_ESTATICLIMIT;
  float* scratch = nullptr;
  const int rc = tb200::static_stab_address(&scratch);
  if (rc != TRITURUS_B200_OK) return rc;
  // Every element the contraction kernel reads is overwritten by the stabiliser pre-pass of the same
  // call, so nothing left behind by an earlier call is ever observed and nothing needs clearing.
  return triturus_b200_lm2exp_f32(a, b, out, R, I, J, K, a_strides, b_strides, out_strides, precision, variant,
                                  scratch, static_cast<size_t>(TRITURUS_B200_STATIC_STAB_FLOATS) * sizeof(float),
                                  status_dev, stream);
}
