/*
 * C ABI of libtriturus_b200.so: the log-space contraction hot path of triturus (lm2exp, lt2exp) as
 * hand-written sm_100a CUDA.  Plain pointers and sizes only; no torch types cross this boundary.
 *
 * All tensor pointers are DEVICE pointers to fp32 data on the device that is current when the call is
 * made.  Strides are in elements.  The innermost stride of every tensor must be 1, every other stride a
 * multiple of 4 elements and every base pointer 16-byte aligned (TMA rules); callers that cannot meet this
 * make a padded copy first (the Python wrappers do).  Exception: the operands a and b of lm2exp may have any
 * strides (zero and negative ones included; the reference forwards whatever it is given,
 * triturus/lm2exp.py:190-198).  Transposed views that otherwise meet the rules (a with i contiguous, b with j
 * contiguous) are read in place through tensor maps, a b of that kind on the single-CTA tiles with the pre-pass
 * stabiliser.  Any other operand that breaks the rules is fetched element by element by the single-CTA kernel
 * (about three times slower per k-block than through TMA: for large problems a padded copy is the faster
 * choice).  Variant codes that ask for a pair tile (or, for a transposed b, the fused max pass) are refused for
 * such operands, and so are returned column maxima together with an element-wise operand.  The library
 * allocates nothing: the output, the
 * workspace and the status word belong to the caller.  Calls are asynchronous on `stream` and never
 * synchronise; they are re-entrant and may run concurrently on different streams or devices as long as
 * each in-flight call has its own workspace and output.
 *
 * Return value: 0 on success or a negative TRITURUS_B200_E* code; nothing is thrown and the process is
 * never terminated.  Device-side protocol time-outs (bounded waits inside the kernels) are reported
 * through `status_dev` (a zero-initialised int32 in device memory, may be NULL): it stays 0 on success and
 * receives a positive code otherwise, readable after the stream has been synchronised.
 */
#ifndef TRITURUS_B200_H
#define TRITURUS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRITURUS_B200_OK 0
#define TRITURUS_B200_EINVAL (-1)      /* bad shape, NULL pointer, unknown precision or variant */
#define TRITURUS_B200_EALIGN (-2)      /* pointer or stride violates the alignment rules above */
#define TRITURUS_B200_EWORKSPACE (-3)  /* workspace too small */
#define TRITURUS_B200_ETENSORMAP (-4)  /* the driver rejected a tensor map */
#define TRITURUS_B200_ELAUNCH (-5)     /* kernel launch or attribute call failed */
#define TRITURUS_B200_EDRIVER (-6)     /* driver entry point unavailable */
#define TRITURUS_B200_ESTATICLIMIT (-7) /* problem exceeds the built-in scratch of the *_static entry point */

#define TRITURUS_B200_PRECISION_TF32 0   /* one tf32 MMA pass; triturus.utils.set_tf32_enabled(True) */
#define TRITURUS_B200_PRECISION_3XTF32 1 /* hi/lo split, ~fp32 accuracy; set_tf32_enabled(False) */

/* Library version, major * 10000 + minor * 100 + patch. */
int triturus_b200_version(void);

/* Human-readable text for a negative return code or a positive status word. */
const char* triturus_b200_strerror(int code);

/*
 * lm2exp: out[r,i,k] = log sum_j a[r,i,j] * exp(b[r,j,k]), stabilised by the clamped column maximum of b
 * so that a column of b that is entirely -inf yields -inf.
 * Replaces triturus/lm2exp.py:167-206 (host wrapper) and :63-164 (_ker_lm2exp); semantics follow
 * baselines/lm2exp.py:4-14.
 *   a [R,I,J], b [R,J,K], out [R,I,K]; *_strides = element strides of the three dimensions.
 *   precision: TRITURUS_B200_PRECISION_*.
 *   variant:   0 = choose everything from the problem size; otherwise STAB * 100000 + BN * 10 + MT with
 *              BN in {128, 256} output columns and MT in {1, 2} 128-row blocks per CTA tile (BN * 10 + MT
 *              may be 0 = automatic; 2564 = a 256 x 256 tile computed by a pair of CTAs, 128 rows each;
 *              2566 = the same tile with the generated operand exp(b - m) kept in tensor memory, plain TF32
 *              only; 2567 = 2566 with the optimistic stabiliser described below)
 *              and STAB selecting where the stabiliser is computed: 0 = automatic, 1 = pre-pass launch
 *              writing the workspace, 2 = max pass fused into the contraction kernel (not with the pair tiles),
 *              3 = that max pass over the first 32 rows of each slab only (optimistic, see below),
 *              4 = pre-pass over the first 32 rows only (optimistic; tile 2564).
 *              (The counterpart of the reference's autotune table, triturus/lm2exp.py:7-58.)
 *   workspace: triturus_b200_lm2exp_workspace_bytes(R, I, J, K) bytes, 256-byte aligned: two flag words padded
 *              to 256 bytes, then the [R,K] stabiliser.  A workspace of only R * K floats is accepted too; the
 *              optimistic stabiliser is then not used.  Keep the workspace between calls (or zero its first
 *              8 bytes once): flag words that are up by accident cost a call the exact passes.
 *
 * Optimistic stabiliser (variant 2567; chosen automatically for plain TF32 on pair tiles, i.e. I > 128, when a has
 * j contiguous and the call has at least 2e10 FLOP): no pre-pass over b.  The contraction kernel takes as
 * stabiliser of a column the maximum over its first 32 rows j; later values may exceed it, exp(b - m) is then
 * larger than 1, which fp32 holds up to e^88.  Only the stabiliser differs from the exact form, so results agree
 * with it to rounding.  A result that overflowed all the same (+inf or NaN) raises the flag word, and the exact
 * form (the same kernel with a max pass over all of b inside) follows in the stream as a launch that returns at
 * once while the flag is down; when it runs it redoes the whole call and its last CTA puts the flag down again (a
 * flag word that is up by accident in fresh memory costs one exact pass).  Inputs whose columns grow by more
 * than ~80 after their first 32 rows therefore cost a second pass.
 * The single-CTA kernel has the same form for its fused max pass (STAB = 3; automatic for plain TF32 when one
 * 128-row block covers I, the contraction has four k-blocks or more, the launch more than one wave of tiles and
 * 2e10 FLOP): the pass scans one k-block instead of the whole slab, and the same kernel with the full pass
 * follows as the conditional launch.  The shared-memory pair kernel (tile 2564; the automatic choice in 3xTF32,
 * with the same size rule) has it as STAB = 4: the pre-pass launch scans 32 rows instead of J, then the
 * contraction and two conditional launches (full pre-pass, contraction), 4 in all.  None of the three is used
 * when column maxima of the result are requested or a stabiliser is supplied.  The reference finds the exact
 * maximum in a first loop over j inside its kernel (triturus/lm2exp.py:124-127).
 */
size_t triturus_b200_lm2exp_workspace_bytes(int64_t R, int64_t I, int64_t J, int64_t K);
/* Number of kernels one triturus_b200_lm2exp_f32 call launches for these arguments on the current device:
 * 2 (stabiliser pre-pass + contraction; or an optimistic kernel + its conditional launch), 1 (fused max pass) or
 * 4 (optimistic 32-row pre-pass, contraction, and two conditional launches; a with j contiguous and a full-size
 * workspace assumed); negative on invalid arguments.  The reference has no counterpart (its launch count is Triton's business, triturus/lm2exp.py:186-205). */
int triturus_b200_lm2exp_launches(int64_t R, int64_t I, int64_t J, int64_t K, int precision, int variant);
int triturus_b200_lm2exp_f32(const float* a, const float* b, float* out, int64_t R, int64_t I, int64_t J, int64_t K,
                             const int64_t a_strides[3], const int64_t b_strides[3], const int64_t out_strides[3],
                             int precision, int variant, void* workspace, size_t workspace_bytes,
                             int32_t* status_dev, void* stream);

/*
 * lm2exp as one link of a chain of layers.  In a circuit the result of one layer is the log-space operand b
 * of the next (the caller's loop around triturus/lm2exp.py:167; the reference recomputes the column maxima of
 * every layer's input inside _ker_lm2exp, triturus/lm2exp.py:124-127).  Here the epilogue of layer n can
 * hand layer n + 1 its stabiliser, so that no layer but the first scans its input for maxima:
 *   b_colmax   (optional) [R,K] contiguous: max_j b[r,j,k], e.g. the out_colmax of the call that produced b,
 *              or the output of triturus_b200_colmax_f32.  Values are clamped to +-1e38 when read.  When
 *              given, no max pass of any kind runs and `workspace` may be NULL.  The result is only
 *              meaningful if the values really are upper bounds close to the column maxima.
 *   out_colmax (optional) [R,K] contiguous: receives max_i out[r,i,k], exactly the maximum of the values
 *              written to out (-inf for a column that is entirely -inf).  The epilogue folds each block of
 *              results into a per-CTA buffer and writes one value per tile column; when the tile has
 *              several row tiles these are reductions into out_colmax, which one small fill launch sets
 *              to -inf first (triturus_b200_lm2exp_chain_launches counts it).
 * With both pointers NULL this is triturus_b200_lm2exp_f32.  variant codes 2xxxxx (fused max pass) are
 * rejected together with b_colmax.
 */
int triturus_b200_lm2exp_chain_launches(int64_t R, int64_t I, int64_t J, int64_t K, int precision, int variant,
                                        int have_b_colmax, int want_out_colmax);
int triturus_b200_lm2exp_chain_f32(const float* a, const float* b, float* out, int64_t R, int64_t I, int64_t J,
                                   int64_t K, const int64_t a_strides[3], const int64_t b_strides[3],
                                   const int64_t out_strides[3], int precision, int variant, const float* b_colmax,
                                   float* out_colmax, void* workspace, size_t workspace_bytes, int32_t* status_dev,
                                   void* stream);

/*
 * lt2exp: out[r,s,k] = log sum_{i,j} w[r,s,i,j] * exp(a[r,i,k]) * exp(b[r,j,k]), stabilised by the clamped
 * column maxima of a and b.
 * Replaces triturus/lt2exp.py:519-630 (host wrapper), :227-357 (_ker_lt2exp_unsplit) and :365-506
 * (_ker_lt2exp_split); semantics follow baselines/lt2exp.py:4-25.
 *   w [R,S,I,J], a [R,I,K], b [R,J,K], out [R,S,K].  w follows the general rules above (it goes through a tensor
 *   map); a and b are read with ordinary loads and may have any strides (triturus/lt2exp.py:580-585, :612-617
 *   forward whatever they are given): 16 bytes at a time when base and strides allow it, else 4.
 *   variant: 0 = automatic, otherwise SPLIT * 10000 + BN * 10 + MT with BN * 10 + MT as above (0 = automatic;
 *            additionally, TF32 only, the generated operand kept in tensor memory instead of shared memory:
 *            1283 / 1284 = tile of 128 columns x 128 / 256 rows, 1285 = 256 columns x 128 rows, which the
 *            automatic choice uses where it would otherwise take 2561)
 *            and SPLIT the number of slices the contraction over (i, j) of every output tile is cut into, the
 *            counterpart of the reference's NUM_SPLITS and mode argument (triturus/lt2exp.py:533-541):
 *            0 = automatic (slices when the output tiles would occupy fewer than half the SMs; when the last
 *            wave of tiles would be less than 90 % full and a tile's contraction is at least 8192 terms long,
 *            the full waves run as whole tiles and the contractions of the last wave's tiles are shared among
 *            all SMs), 1 = never (mode "unsplit"), n >= 2 = n slices (fewer if a slice would drop below 16
 *            k-blocks), 9998 = the shared last wave in any case, 9999 = as automatic but at least two slices
 *            (mode "split").  Plain TF32 over more than 32768 terms re-sums its accumulator every 4096
 *            terms with rounded adds (automatic tiles only leave room for that; an explicit 2562 / 128x tile is
 *            honoured and runs without).  A split call launches three kernels: zero-fill
 *            of out, the slices adding their partial sums into out with fp32 reductions (so the last bits
 *            depend on arrival order, as they do under the reference's spin lock, triturus/lt2exp.py:498-506),
 *            and the in-place log pass.  Unsplit results are deterministic.
 *   No workspace is needed.
 */
/* Number of kernels one triturus_b200_lt2exp_f32 call launches for these arguments on the current device
 * (1, or 3 when the contraction is split); negative on invalid arguments. */
int triturus_b200_lt2exp_launches(int64_t R, int64_t S, int64_t I, int64_t J, int64_t K, int precision, int variant);
/* What a triturus_b200_lt2exp_f32 call with these arguments runs on the current device, as the explicit variant
 * code that pins it: SPLIT * 10000 + BN * 10 + MT with SPLIT = 1 (whole tiles), the slice count, or 9998 (last
 * wave shared).  The counterpart of reading the reference's autotuner choice (triturus/lt2exp.py:9-75,78-222); negative
 * on invalid arguments. */
int triturus_b200_lt2exp_plan(int64_t R, int64_t S, int64_t I, int64_t J, int64_t K, int precision, int variant);
/* The same for triturus_b200_lm2exp_f32: STAB * 100000 + BN * 10 + MT with STAB = 1 (pre-pass), 2 (fused max
 * pass), 3 or 4 (their optimistic forms); the tile code 2567 stands by itself (its stabiliser is part of the
 * tile).  Negative on invalid arguments. */
int triturus_b200_lm2exp_plan(int64_t R, int64_t I, int64_t J, int64_t K, int precision, int variant);
int triturus_b200_lt2exp_f32(const float* w, const float* a, const float* b, float* out, int64_t R, int64_t S,
                             int64_t I, int64_t J, int64_t K, const int64_t w_strides[4], const int64_t a_strides[3],
                             const int64_t b_strides[3], const int64_t out_strides[3], int precision, int variant,
                             int32_t* status_dev, void* stream);
/*
 * The same with caller-provided scratch memory, the counterpart of the lock tensor the reference's wrapper
 * allocates for its split kernel (triturus/lt2exp.py:555-562).  With it the shared last wave (SPLIT 9998, and the
 * automatic choice for a ragged last wave) needs one launch and no atomics: a CTA that works on a later part of
 * a tile's contraction parks its raw partial sums in the workspace, and the CTA that holds the tile's first
 * k-blocks adds them to its own and writes the finished results.  The order of those additions is fixed, so
 * the results do not depend on timing.  triturus_b200_lt2exp_f32 (no workspace) never chooses the shared last
 * wave by itself and, when asked for it, falls back to additions into the zero-filled result.
 *   workspace: triturus_b200_lt2exp_workspace_bytes(...) bytes, 256-byte aligned (0 bytes: may be NULL); its
 *   first 1024 bytes are cleared by a cudaMemsetAsync on `stream` in every call that uses it.  The queries
 *   triturus_b200_lt2exp_launches / _plan describe calls of this entry point with that workspace.
 *   The CTAs of such a launch wait for one another (with the usual bound), so the launch takes the whole GPU:
 *   on a device that another kernel shares at the same time, a CTA may start late and a wait may run out
 *   (reported through status_dev, never a hang).
 */
size_t triturus_b200_lt2exp_workspace_bytes(int64_t R, int64_t S, int64_t I, int64_t J, int64_t K, int precision,
                                            int variant);
int triturus_b200_lt2exp_ws_f32(const float* w, const float* a, const float* b, float* out, int64_t R, int64_t S,
                                int64_t I, int64_t J, int64_t K, const int64_t w_strides[4],
                                const int64_t a_strides[3], const int64_t b_strides[3], const int64_t out_strides[3],
                                int precision, int variant, void* workspace, size_t workspace_bytes,
                                int32_t* status_dev, void* stream);

/*
 * lt2exp as one link of a chain of layers (see triturus_b200_lm2exp_chain_f32; the reference's kernels scan a
 * and b for their column maxima in every call, triturus/lt2exp.py:305-311).
 *   a_colmax, b_colmax (optional, both or neither) [R,K] contiguous: max_i a[r,i,k] and max_j b[r,j,k], e.g.
 *              the out_colmax of the calls that produced a and b.  Clamped to +-1e38 when read; when given,
 *              the kernels do not scan a and b.
 *   out_colmax (optional) [R,K] contiguous: receives max_s out[r,s,k], exactly the maximum of the values
 *              written to out; costs one small fill launch (one more than triturus_b200_lt2exp_launches
 *              reports) and a reduction in the epilogue, or in the log pass of a split contraction.
 * With all three NULL this is triturus_b200_lt2exp_f32.
 */
int triturus_b200_lt2exp_chain_f32(const float* w, const float* a, const float* b, float* out, int64_t R, int64_t S,
                                   int64_t I, int64_t J, int64_t K, const int64_t w_strides[4],
                                   const int64_t a_strides[3], const int64_t b_strides[3],
                                   const int64_t out_strides[3], int precision, int variant, const float* a_colmax,
                                   const float* b_colmax, float* out_colmax, int32_t* status_dev, void* stream);

/*
 * The stabiliser alone: m[r,k] = clamp(max_j x[r,j,k], -1e38, 1e38), m contiguous [R,K].
 * This is the pre-pass of triturus/lm2exp.py:125-127 (and baselines/lm2exp.py:11-12) as its own launch.
 */
int triturus_b200_colmax_f32(const float* x, float* m, int64_t R, int64_t J, int64_t K, const int64_t x_strides[3],
                             void* stream);

/*
 * Plain matrix product out[M,N] = a[M,K] * b[K,N] through the same pipeline with the log-space steps switched off.
 * Replaces triturus/mm.py:181-214 (wrapper) and :91-178 (_ker_mm).  precision TF32: both operands rounded to the
 * nearest tf32, as the reference's kernel does with cvt.rna (triturus/mm.py:152-154, triturus/utils.py:56-63);
 * precision 3XTF32: the hi/lo split, ~fp32 accuracy (the reference's "ieee" dot).  Strides in elements, innermost
 * stride 1, row strides multiples of 4 elements, bases 16-byte aligned.  No workspace.  Inf / NaN inputs are not
 * supported in TF32 mode (the rounding is done on the bit pattern).
 */
int triturus_b200_mm_f32(const float* a, const float* b, float* out, int64_t M, int64_t K, int64_t N,
                         const int64_t a_strides[2], const int64_t b_strides[2], const int64_t out_strides[2],
                         int precision, int32_t* status_dev, void* stream);

/*
 * Self-test of the error path behind `status_dev` (no counterpart in the reference, whose kernels have no waits
 * that could time out apart from the unbounded spin lock of triturus/lt2exp.py:498-506).  Launches one 64-thread
 * block in which a warp waits on a barrier that nobody signals, with a wait limit of `limit_cycles` GPU clock
 * cycles (1e3 ... 2e8, i.e. at most ~0.1 s) instead of the ~1.5 s the kernels use.  The wait gives up, the other
 * warp of the block leaves its own wait on seeing the abort flag, and the kernel returns by itself with the code
 * 105 ("device: setup wait timed out") in *status_dev.  Nothing traps, faults or spins without a bound.
 */
int triturus_b200_selftest_wait_timeout(int32_t* status_dev, int64_t limit_cycles, void* stream);

/*
 * lm2exp for callers that cannot allocate device memory.  (No counterpart in the reference: its wrapper
 * allocates freely through torch.)
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- inside an arena or memory pool that already
 * owns the GPU's memory, in latency-critical loops where an allocation would synchronise the device, or in
 * plugin hosts that pass in only the input and output buffers.  Same arguments and results as
 * triturus_b200_lm2exp_f32, minus the workspace: the [R,K] stabiliser scratch is a fixed 4 MiB array inside
 * the library image (reserved on every GPU that loads the library, until the process exits).
 *
 *   Limit:  R * K <= triturus_b200_lm2exp_static_max_columns() (1,048,576); larger problems return
 *           TRITURUS_B200_ESTATICLIMIT and launch nothing.
 *   Set-up: the first call on each device looks up the array's device address (that device must be
 *           current); make that first call before starting any stream capture.
 *   Sharing: all calls on a device use the same array.  Each call rewrites every element it later reads, so
 *           stale contents never matter, but two calls whose kernels can overlap on the GPU (different
 *           streams, no dependency) race on it; keep such calls ordered or use the workspace entry point.
 *   The function calls no cudaMalloc, cudaFree or any other allocating routine.
 */
size_t triturus_b200_lm2exp_static_max_columns(void);
int triturus_b200_lm2exp_f32_static(const float* a, const float* b, float* out, int64_t R, int64_t I, int64_t J,
                                    int64_t K, const int64_t a_strides[3], const int64_t b_strides[3],
                                    const int64_t out_strides[3], int precision, int variant, int32_t* status_dev,
                                    void* stream);

#ifdef __cplusplus
}
#endif

#endif /* TRITURUS_B200_H */
