// Thin inline-PTX wrappers for the sm_100a features the contraction kernels use:
// mbarrier (with bounded waits), TMA tiled loads, tcgen05 (TMEM alloc, MMA, commit, ld) and
// the proxy / tcgen05 fences that order them.
//
// Every wait in this file is bounded: a wait that runs past WAIT_LIMIT_CYCLES raises the CTA's
// abort flag, records an error code in the launch's status word and returns false.  Callers
// leave their loops on `false`, meet at the CTA's final barrier and free TMEM, so a
// protocol bug ends as an error code on the host and never as a hung GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb200 {

// ~1.5 s at 1.9 GHz.  Legitimate waits are tens of microseconds.
constexpr long long WAIT_LIMIT_CYCLES = 3000000000LL;

// Error codes written to the status word (first failure wins).
enum StatusCode : int {
  STATUS_OK = 0,
  STATUS_TIMEOUT_PRODUCER = 101,
  STATUS_TIMEOUT_TRANSFORM = 102,
  STATUS_TIMEOUT_MMA = 103,
  STATUS_TIMEOUT_EPILOGUE = 104,
  STATUS_TIMEOUT_SETUP = 105,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ----------------------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// True in exactly one lane of a fully converged warp (the same lane on every call).  Code that the whole warp
// runs with uniform control flow and that issues its single-thread instructions under this predicate keeps
// its addresses and descriptors in uniform registers.
__device__ __forceinline__ bool elect_one_sync() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}"
      : "=r"(pred));
  return pred != 0;
}

// Per-CTA abort state shared by all roles.
struct AbortCtl {
  volatile int* flag;   // shared memory, set once any wait gives up
  int* status;          // global status word of the launch (may be nullptr)
};

__device__ __forceinline__ void raise_abort(const AbortCtl& ctl, int code) {
  *ctl.flag = 1;
  if (ctl.status != nullptr) atomicCAS(ctl.status, 0, code);
}

// Bounded wait on one phase of an mbarrier.  Returns false if the CTA is aborting.  `limit` is the number of
// clock cycles after which the wait gives up (the kernels use WAIT_LIMIT_CYCLES; the self-test passes a short one).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const AbortCtl& ctl, int code,
                                          long long limit = WAIT_LIMIT_CYCLES) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*ctl.flag) return false;
    if (clock64() - t0 > limit) {
      raise_abort(ctl, code);
      return false;
    }
  }
}

// Same wait, made warp-uniform: either every lane sees the phase complete or every lane leaves.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, const AbortCtl& ctl, int code,
                                               long long limit = WAIT_LIMIT_CYCLES) {
  const bool ok = mbar_wait(bar, parity, ctl, code, limit);
  return __all_sync(0xffffffffu, ok);
}

// ----------------------------------------------------------------------------- 4-byte asynchronous copies
//
// For operands that a tensor map cannot describe (rows that do not start on 16-byte boundaries, an innermost
// stride other than 1): one element per copy, zeros where `valid` is false (the source is then not read).
__device__ __forceinline__ void cp_async_f32(uint32_t smem_dst, const float* src, bool valid) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_dst), "l"(src), "r"(valid ? 4 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------- CTA pairs (clusters of two)

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// All threads of all CTAs of the cluster.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of the same shared-memory object in the CTA with rank `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

// Arrive on an mbarrier that may live in the other CTA of the pair.  What the waiter consumes afterwards
// moves through the async proxy (TMA-written tiles, operands read by the tensor core after
// fence.proxy.async), so the barrier's own ordering suffices and no cluster-scope fence is paid per k-block.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// ----------------------------------------------------------------------------- flags in global memory
//
// Hand-over between CTAs of one launch: the writer makes its data visible (__threadfence) and raises a counter
// with release semantics; the reader polls the counter with acquire semantics (always with a bound on the
// number of polls or cycles) and then reads the data with ordinary, not read-only-path, loads.
__device__ __forceinline__ void add_release_gpu(int* addr, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* addr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// ----------------------------------------------------------------------------- programmatic dependent launch
//
// A kernel launched with cudaLaunchAttributeProgrammaticStreamSerialization may start while the kernel before
// it in the stream is still running, once every block of that kernel has called pdl_launch_dependents() or
// exited.  Its threads must call pdl_wait() before they touch anything the earlier kernel writes; the call
// returns when that kernel has completed and its writes are visible.  Both are no-ops in a kernel launched the
// ordinary way.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ----------------------------------------------------------------------------- fences

// Generic-proxy shared-memory writes -> visible to the async proxy (TMA, tcgen05.mma operands).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ----------------------------------------------------------------------------- TMA (no multicast anywhere)

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 3-D tiled load global -> this CTA's shared memory; completion counted in bytes on `bar`.
// x is the innermost coordinate and must keep x * 4 bytes a multiple of 16.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y,
                                            int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z),
      "r"(w)
      : "memory");
}

// Bring a 3-D box into L2 only (no shared-memory destination, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_l2_3d(const CUtensorMap* tmap, int x, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(x), "r"(y), "r"(z)
               : "memory");
}

// 3-D tiled store shared memory -> global (bulk async group).  Elements of the box that fall outside the
// tensor are not written.  The shared-memory source must stay untouched until tma_store_wait_read().
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tmap, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// All but the newest `N` bulk groups of this thread have finished READING their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// All bulk groups of this thread are complete (their global writes are done).
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ----------------------------------------------------------------------------- TMEM

// Whole-warp collectives.  ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// The same for a CTA pair: executed by the same warp of both CTAs, allocates the same columns in both.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// 32 lanes x 32 consecutive columns: lane l of the warp receives columns [c, c+32) of TMEM lane
// (lane field of taddr) + l.  A warp may only touch the lane quarter 32 * (warp_id % 4).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// Registers -> TMEM, the inverse of tmem_ld_32x32: lane l of the warp writes 32 consecutive columns of TMEM
// lane (lane field of taddr) + l.
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
      "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
      "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------- tcgen05.mma (TF32, operands in smem)

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes (32 fp32) wide and
// stored with the 128-byte swizzle (16-byte chunk index XOR row % 8); 8-row groups are 1024 bytes apart.
// The tile base must be 1024-byte aligned.  Advancing the contraction index by 8 elements (one
// MMA) adds 32 bytes, i.e. 2 to the encoded start address.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset: unused for swizzled K-major
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version of this architecture
  d |= static_cast<uint64_t>(2) << 61;                      // 128-byte swizzle
  return d;
}

// Shared-memory matrix descriptor for an MN-major tf32 operand.  The only swizzled layout the tensor core
// accepts for 32-bit MN-major operands is the 128-byte swizzle with a 32-byte base: rows of 32 consecutive
// MN elements (128 bytes) per contraction index, 128 bytes apart, in atoms of 4 rows (512 bytes) inside which
// the 32-byte chunk index is XORed with row % 4 (address bits [5,7) ^= bits [7,9)).  TMA writes exactly this
// pattern with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.  Consecutive 32-element MN groups are
// `group_stride_bytes` apart (leading byte offset); consecutive 4-row atoms are 512 bytes apart (stride byte
// offset).  One MMA (8 contraction values) spans two atoms, so advancing the contraction index by 8 adds
// 1024 bytes, i.e. 64 to the encoded start address.  Used with bit 16 (B is MN-major) set in the instruction
// descriptor.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128_base32(uint32_t smem_addr, uint32_t group_stride_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((group_stride_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>(512 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(1) << 61;  // 128-byte swizzle, 32-byte base
  return d;
}

// Byte offset of the 16-byte chunk `c` (0..7) of row `j` inside a box of 128-byte rows stored with the
// 128-byte / 32-byte-base swizzle.
__device__ __forceinline__ uint32_t sw128_base32_offset(uint32_t j, uint32_t c) {
  return j * 128u + (((((c >> 1) ^ (j & 3u)) << 1) | (c & 1u)) << 4);
}

// Instruction descriptor: D = fp32, A = B = tf32, both K-major, dense, no negate.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// One MMA D[tmem] (+)= A[smem] * B[smem], issued by a single thread.
__device__ __forceinline__ void umma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Pair MMA: issued by one thread of the leader CTA, executed by the tensor cores of both CTAs.  With
// M = 256 each CTA supplies its own 128 rows of A and its own half of the N columns of B from the same
// shared-memory offsets, and receives its 128 rows of D in its own TMEM.
__device__ __forceinline__ void umma_tf32_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive on the mbarrier at `cluster_addr` (this CTA's or, through map_to_cta, the other CTA's) once every
// pair MMA issued so far by this thread has finished in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

// The same arrival delivered to the mbarrier at this shared-memory offset in every CTA of `cta_mask`
// (bit i = CTA rank i): one instruction frees a stage in both CTAs of a pair.
__device__ __forceinline__ void umma_commit_pair_mcast(uint32_t smem_addr, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_addr),
      "h"(cta_mask)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from TMEM (lane = row of A, one 32-bit column per
// contraction index, always K-major); B comes from shared memory through its descriptor.
__device__ __forceinline__ void umma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive on `bar` once every MMA issued so far by this thread has finished (implies
// tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ----------------------------------------------------------------------------- math helpers

constexpr float LOG2E_F = 1.4426950408889634f;
constexpr float LN2_F = 0.6931471805599453f;
constexpr float STAB_CLAMP = 1e38f;  // the reference clamps the stabiliser to +-1e38 (baselines/lm2exp.py:12)

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// exp(v - m) with the subtraction done first, as the reference does (baselines/lm2exp.py:13).
__device__ __forceinline__ float exp_shifted(float v, float m) { return ex2_approx((v - m) * LOG2E_F); }

// Round an fp32 in [0, +inf) to the nearest tf32 (ties away), as raw bits.  The tensor core drops the low
// 13 mantissa bits of its operands, so adding half a tf32 ulp beforehand turns that truncation into
// rounding.  Not valid for inf/nan.
__device__ __forceinline__ uint32_t tf32_round_bits(float x) { return __float_as_uint(x) + 0x1000u; }

// Exact hi/lo split for the 3xTF32 scheme: hi has only tf32 bits set, lo = x - hi is exact in fp32.
__device__ __forceinline__ void tf32_split_rn(float x, float& hi, float& lo) {
  hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
  lo = x - hi;
}
__device__ __forceinline__ void tf32_split_trunc(float x, float& hi, float& lo) {
  hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
  lo = x - hi;
}

// Four fp32 additions into global memory with one reduction instruction (address 16-byte aligned).
__device__ __forceinline__ void red_add_f32x4(float* addr, float x, float y, float z, float w) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}

__device__ __forceinline__ float clamp_stab(float m) { return fminf(fmaxf(m, -STAB_CLAMP), STAB_CLAMP); }

// ----------------------------------------------------------------------------- column maxima of the result
//
// An epilogue that also returns m[k] = max_i out[i, k] folds every 32 x 32 block of results into a per-CTA
// buffer in shared memory (one word per tile column, all four epilogue warps and all row blocks of the tile),
// and writes the buffer to global memory once per tile.  Floats are kept as their bit patterns: non-negative
// floats order like signed integers and negative floats in reverse like unsigned integers, so an integer
// max / min does a float max whatever the sign of the stored value.  NaN does not occur.

constexpr int NEG_INF_BITS = static_cast<int>(0xFF800000u);

__device__ __forceinline__ void smem_max_f32(int* addr, float v) {
  v += 0.f;  // -0 becomes +0, whose bit pattern orders correctly
  if (v >= 0.f) atomicMax(addr, __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned*>(addr), __float_as_uint(v));
}

__device__ __forceinline__ void red_max_f32(float* addr, float v) {
  v += 0.f;
  if (v >= 0.f) {
    asm volatile("red.global.max.s32 [%0], %1;" ::"l"(addr), "r"(__float_as_int(v)) : "memory");
  } else {
    asm volatile("red.global.min.u32 [%0], %1;" ::"l"(addr), "r"(__float_as_uint(v)) : "memory");
  }
}

// Block held one row per lane (o[e] = column e of row `lane`): returns in lane c the maximum of column c over
// the rows with row_valid.  Transposing reduction: at distance d a lane keeps the half of its columns whose
// index has bit d equal to its own lane bit and trades the other half with lane ^ d, so five rounds
// (16 + 8 + 4 + 2 + 1 shuffles) do it.
__device__ __forceinline__ float block_colmax_to_lanes(const float (&o)[32], bool row_valid, int lane) {
  float v[32];
#pragma unroll
  for (int e = 0; e < 32; ++e) v[e] = row_valid ? o[e] : -INFINITY;
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) {
    const bool upper = (lane & d) != 0;
#pragma unroll
    for (int e = 0; e < d; ++e) {
      const float keep = upper ? v[e + d] : v[e];
      const float send = upper ? v[e] : v[e + d];
      v[e] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, d));
    }
  }
  return v[0];
}

// The same from the 32 x 32 staging box the epilogue has just written for its TMA store (row r at byte
// r * 128, 16-byte chunk g at position g ^ (r % 8)): eight 16-byte loads give a lane 8 rows of 4 columns, which
// it folds in registers; two shuffle rounds fold the four row slots of the warp.  A third of the instructions
// of block_colmax_to_lanes.  The caller has synchronised the warp after the writes.
// `box_free` (optional): an mbarrier on which one lane arrives as soon as every lane holds its part of the
// box in registers, for a caller that reads the box on behalf of the warp that wants to overwrite it.
__device__ __forceinline__ void fold_staged_colmax(const uint8_t* stg, int rows_valid, int* cb, int lane,
                                                   uint64_t* box_free = nullptr) {
  const int g = lane & 7, rs = lane >> 3;
  float4 mx = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = rs + 4 * i;
    const float4 v = *reinterpret_cast<const float4*>(stg + r * 128 + ((g ^ (r & 7)) << 4));
    if (r < rows_valid) {
      mx.x = fmaxf(mx.x, v.x);
      mx.y = fmaxf(mx.y, v.y);
      mx.z = fmaxf(mx.z, v.z);
      mx.w = fmaxf(mx.w, v.w);
    }
  }
  if (box_free != nullptr) {
    __syncwarp();  // the shuffles below would do, but the hand-back must not depend on their placement
    if (lane == 0) mbar_arrive(box_free);
  }
#pragma unroll
  for (int sh = 8; sh <= 16; sh <<= 1) {
    mx.x = fmaxf(mx.x, __shfl_xor_sync(0xffffffffu, mx.x, sh));
    mx.y = fmaxf(mx.y, __shfl_xor_sync(0xffffffffu, mx.y, sh));
    mx.z = fmaxf(mx.z, __shfl_xor_sync(0xffffffffu, mx.z, sh));
    mx.w = fmaxf(mx.w, __shfl_xor_sync(0xffffffffu, mx.w, sh));
  }
  if (rs == 0) {
    smem_max_f32(cb + g * 4 + 0, mx.x);
    smem_max_f32(cb + g * 4 + 1, mx.y);
    smem_max_f32(cb + g * 4 + 2, mx.z);
    smem_max_f32(cb + g * 4 + 3, mx.w);
  }
}

// Rows 0..nrows-1 of a staged 32 x 32 box to global memory, lane = column: every store instruction of the
// warp writes 32 consecutive floats of one row (`dst` points at this lane's column of row 0).  For results
// that cannot go through a TMA store.  Kept out of line: inlined, its address arithmetic competes for
// registers with the accumulator chunks the epilogue holds.
__device__ __noinline__ void store_staged_rows(const uint8_t* stg, float* dst, int64_t row_stride, int nrows,
                                               int lane) {
  const uint8_t* src = stg + (lane & 3) * 4;
#pragma unroll 4
  for (int rr = 0; rr < 32; ++rr) {
    if (rr < nrows)
      dst[static_cast<int64_t>(rr) * row_stride] =
          *reinterpret_cast<const float*>(src + rr * 128 + (((lane >> 2) ^ (rr & 7)) << 4));
  }
}

// End of a tile, called by the two fold warps after they have met at a barrier: thread te of 64 moves
// columns te, te + 64, ... of the tile's buffer to gcol (a plain store when this tile alone covers the
// column, else a reduction with the other row tiles) and resets the buffer.
__device__ __forceinline__ void flush_tile_colmax(int* cb, int bn, float* gcol, int ncols_valid, bool exclusive,
                                                  int te) {
  for (int c = te; c < bn; c += 64) {
    const float v = __int_as_float(cb[c]);
    cb[c] = NEG_INF_BITS;
    if (c < ncols_valid) {
      if (exclusive) gcol[c] = v;
      else red_max_f32(gcol + c, v);
    }
  }
}

// Byte offset of element (row, col) inside a 128-byte-swizzled K-major tile (rows of 32 fp32).
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t col) {
  return row * 128u + ((((col >> 2) ^ (row & 7u)) << 4) | ((col & 3u) << 2));
}

}  // namespace tb200
