/*
 * fp8mm_b200.h — C ABI of the B200 (sm_100a) block-scaled FP8 GEMM library.
 *
 *   C[M,N] (bf16) = sum_kb ( A_e4m3[M, 128kb..] . B_e4m3[N, 128kb..]^T ) * As[M,kb] * Bs[N/128,kb]
 *
 * This is the boundary a foreign-function binding attaches to.  It replaces the
 * kernel registry and the per-kernel host wrappers of the reference project:
 *   fp8_gemm_h20/engine.py:5-19            (name -> kernel, run(entry, args))
 *   fp8_gemm_h20/kernels/kernel_v2.py:339-376   (config merge, split legalisation,
 *                                           workspace, output allocation, launch)
 *   fp8_gemm_h20/kernels/baseline_gluon.py:259-293, baseline_triton.py:87-114,
 *   kernel_scale_tma.py:356-396, kernel_shortk.py:46-54   (the other wrappers)
 *
 * Plain pointers and sizes only: no torch types, no C++ types.  Every function
 * returns 0 on success or a negative FP8MM_E_* code; nothing throws, traps or
 * aborts.  All launches are asynchronous on the stream that is passed in.
 */
#ifndef FP8MM_B200_H_
#define FP8MM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error codes -------------------------------------------------------- */
#define FP8MM_OK                0
#define FP8MM_E_NULL           -1   /* a required pointer is NULL                      */
#define FP8MM_E_SHAPE          -2   /* M<1, or N or K not a multiple of 128            */
#define FP8MM_E_CONFIG         -3   /* tile / split / stage combination not legal      */
#define FP8MM_E_WORKSPACE      -4   /* workspace missing or smaller than required      */
#define FP8MM_E_ALIGN          -5   /* A or B not 16-byte aligned, C not 16-byte aligned */
#define FP8MM_E_DRIVER         -6   /* tensor-map encode or another driver call failed */
#define FP8MM_E_LAUNCH         -7   /* the kernel launch itself was refused            */
#define FP8MM_E_DEVICE_TIMEOUT -8   /* a bounded device-side wait gave up (see status) */
#define FP8MM_E_TOO_LARGE      -9   /* needs more scratch than the built-in buffer of the
                                       allocation-free entry point holds                   */

/* ---- kernel families ("impl" names of the JSON tuning tables) ------------ */
#define FP8MM_IMPL_UMMA        0    /* tokens on the 128 UMMA rows, weights on UMMA-N (128|256)  */
#define FP8MM_IMPL_UMMA_SWAP   1    /* swap-AB: weights on the 128 UMMA rows, tokens on UMMA-N   */
#define FP8MM_IMPL_UMMA_2CTA   2    /* CTA pairs (cta_group::2): 256 tokens x 256 weights per pair */
#define FP8MM_IMPL_GEMV        3    /* decode (one to a handful of tokens): weight rows streamed straight
                                       into registers, FP32 FMAs, 8 weight rows x 512 bytes of K per warp
                                       step; no tensor memory, no barriers, no tensor maps.  Successor of
                                       the reference's smallest tiles (BT=8, BW=16..128, kernel_v2.py:94-291
                                       with the M<=8 entries of configs/122b_tp4.json)               */
#define FP8MM_IMPL_UMMA_MX     4    /* power-of-two scales applied by the tensor cores themselves
                                       (tcgen05.mma kind::mxf8f6f4.block_scale): As and Bs point to UE8M0
                                       BYTES (value 2^(b-127); strides in bytes), FP32 accumulation over
                                       the K range in tensor memory.  The native form of the reference
                                       adapter's DEEPGEMM_SCALE_UE8M0 mode (sgl_patch/fp8mm_sglang_patch.py).
                                       (block_t, block_w) = (128, 256) or (256, 224) token-major tiles (no
                                       split-K), or (16|32|64|128, 128) swap-AB tiles for up to a few hundred
                                       tokens; these take cfg.split like the table kernels (cluster
                                       reduction for 2, 4, 8, the workspace otherwise; a split that does not
                                       divide K/128 runs unsplit)                                        */

/* cfg.flags: reduce split-K partials through the global workspace even where the cluster
 * (distributed shared memory) reduction is available (splits of 2, 4 and 8). */
#define FP8MM_FLAG_WORKSPACE_SPLIT 1
/* cfg.flags: two K blocks per shared-memory ring slot, fetched by one 3-D TMA copy per operand
 * (swap-AB tiles of 16..64 tokens; needs an even number of K blocks per split, otherwise ignored).
 * Halves the per-K-block work of the single TMA-issuing thread, which paces small-M calls.
 * With FP8MM_IMPL_UMMA_MX swap-AB tiles of 16..64 tokens (unsplit): the half-size form, two K blocks per slot
 * and two MMA-issuing threads instead of four, half the tensor memory, so that two CTAs share an SM; pays
 * where the work units outnumber the SMs.  Accumulation order differs from the full-size form (two partial
 * sums instead of four), the result stays within the same tolerance. */
#define FP8MM_FLAG_K_PAIRS 2
/* cfg.flags bits 8..11: K blocks per ring slot, 2..8 (table key K_GROUP); generalises FP8MM_FLAG_K_PAIRS.
 * Needs the count to divide the K blocks of every split and two such slots to fit in shared
 * memory, otherwise ignored.  The result bits do not depend on it. */
#define FP8MM_FLAG_K_GROUP(n) (((n) & 15) << 8)
#define FP8MM_FLAG_K_GROUP_MASK 0xF00
/* cfg.flags, FP8MM_IMPL_GEMV: As and Bs point to UE8M0 exponent bytes (value 2^(b-127); strides in bytes)
 * instead of floats, as they always do for FP8MM_IMPL_UMMA_MX (where the flag is accepted and redundant). */
#define FP8MM_FLAG_SCALES_UE8M0 4
/* cfg.flags, with exponent-byte scales (FP8MM_IMPL_UMMA_MX, or FP8MM_IMPL_GEMV with the flag above): As holds
 * float32 powers of two after all (strides in elements), as a quantiser with power-of-two scales hands them
 * over (SGLang's with scale_ue8m0=True); the kernels take the exponent field.  Bs stays bytes. */
#define FP8MM_FLAG_ACT_SCALES_F32 8

/*
 * Operands.  Strides are in ELEMENTS and are exactly the values the reference
 * hands to its kernels (kernel_v2.py:371-372: As.stride(0), As.stride(1),
 * Bs.stride(0), Bs.stride(1)); ldc is new so that an N-shard can write into a
 * column slice of a wider C.
 *   A  [M,K]      float8_e4m3fn, row-major, contiguous (ld = K)     dispatch.py:22
 *   B  [N,K]      float8_e4m3fn, row-major, contiguous (ld = K)     dispatch.py:22
 *   As [M,K/128]  float32, any strides                              dispatch.py:24-27
 *   Bs [N/128,K/128] float32, any strides                           dispatch.py:24-27
 *   C  [M,N]      bfloat16, row stride ldc >= N
 */
typedef struct fp8mm_args {
  const void*  A;
  const void*  B;
  const float* As;
  const float* Bs;
  void*        C;
  int32_t      M, N, K;
  int32_t      reserved0;
  int64_t      as_stride_m, as_stride_k;
  int64_t      bs_stride_n, bs_stride_k;
  int64_t      ldc;
} fp8mm_args;

/*
 * Launch configuration = one "config" object of a tuning-table entry
 * (fp8_gemm_h20/configs/*.json, "entries"/"N,K"/"M"/{"impl","config"}).
 *   block_t   token tile   (BLOCK_T):  UMMA   -> 128;  UMMA_SWAP -> 16,32,64,128,256;  UMMA_2CTA -> 256;
 *             GEMV -> 1, 2 or 4 tokens per warp (more tokens run as further token groups)
 *   block_w   weight tile  (BLOCK_W):  UMMA   -> 128 or 256;  UMMA_SWAP -> 128;  UMMA_2CTA -> 256;  GEMV -> 8
 *   stages    depth of the TMA shared-memory ring (NUM_STAGES); clipped to what fits
 *   split     split-K factor (SPLIT); a value that does not divide K/128 is
 *             legalised to 1, as the reference wrapper does (kernel_v2.py:355-356)
 *   group_m   token tiles per raster group (GROUP_SIZE_M), >=1
 *   max_ctas  0 = one wave sized from the SM count; otherwise an upper bound on the grid
 * A cluster launch needs room for `split` co-scheduled CTAs; where the context has none (an
 * SM-limited or partitioned context) the call falls back to the workspace reduction if the
 * workspace passed in is large enough for it (ask fp8mm_b200_workspace_bytes with
 * FP8MM_FLAG_WORKSPACE_SPLIT set), else it returns FP8MM_E_WORKSPACE.
 * Split-K partials are reduced in split order, either by the CTA that arrives last on a
 * per-tile counter (workspace path, kernel_v2.py:274-289) or, for splits of 2, 4 and 8, by the
 * `split` CTAs of the tile themselves, launched as one thread-block cluster and reading each
 * other's shared memory (no workspace traffic); both give the same bits.
 */
typedef struct fp8mm_cfg {
  int32_t impl;
  int32_t block_t;
  int32_t block_w;
  int32_t stages;
  int32_t split;
  int32_t group_m;
  int32_t max_ctas;
  int32_t flags;      /* 0, or FP8MM_FLAG_* bits */
} fp8mm_cfg;

/* Legality of (M,N,K,cfg) without touching the GPU.  Replaces the per-wrapper
 * asserts (kernel_v2.py:341-349, kernel_shortk.py:49) and the tile checks of
 * config.py:44-56.  Returns FP8MM_OK or a negative code. */
int fp8mm_b200_validate(int32_t M, int32_t N, int32_t K, const fp8mm_cfg* cfg);

/* Bytes of zero-initialised device workspace the call needs (status words,
 * split-K tile counters and fp32 partial tiles).  Replaces the per-(device,
 * stream) workspace sizing of kernel_v2.py:309-324.  The same workspace must not
 * be used by two launches that can overlap on the GPU: keep one per stream. */
size_t fp8mm_b200_workspace_bytes(int32_t M, int32_t N, int32_t K, const fp8mm_cfg* cfg);

/* Zero a fresh workspace on `stream` (a cudaStream_t).  Needed once after
 * allocation; the kernels leave the counters at zero again after every launch
 * (kernel_v2.py:289 does the same with atomic_xchg), so graph replay is safe. */
int fp8mm_b200_workspace_init(void* workspace, size_t ws_bytes, void* stream);

/* Enqueue one GEMM on `stream` (a cudaStream_t) of the current device.
 * Replaces engine.run -> block_fp8_gemm_* (engine.py:18-19, kernel_v2.py:339-376).
 * Inputs are borrowed until the enqueued work has run; nothing is allocated. */
int fp8mm_b200_gemm(const fp8mm_args* args, const fp8mm_cfg* cfg,
                    void* workspace, size_t ws_bytes, void* stream);

/* The same GEMM with its result also stored into up to 7 more buffers of the same shape and
 * row stride: `extra_c[i]` are device pointers, typically the peer GPUs' copies of the output
 * of an N-sharded (column-parallel) layer, mapped into this process (CUDA IPC / symmetric
 * memory).  The kernel's epilogue writes every tile to args->C and to each extra target with
 * plain peer-to-peer stores, which fuses the all-gather that would otherwise follow the GEMM.
 * The caller orders the peers' reads after this kernel (a barrier across the ranks).
 * No counterpart in the reference, which is single-GPU (README.md:50,74). */
int fp8mm_b200_gemm_bcast(const fp8mm_args* args, const fp8mm_cfg* cfg, void* workspace, size_t ws_bytes,
                          void* stream, void* const* extra_c, int32_t n_extra);

/*
 * Allocation-free variant of fp8mm_b200_gemm.  No counterpart in the reference: its wrappers
 * allocate their split-K workspace with torch (kernel_v2.py:316-324) and so does the binding
 * that ships with this library.
 *
 * Who needs it: hosts that must not (or cannot) call cudaMalloc on the GEMM path — an inference
 * server that has handed every byte of device memory to its own pool allocator at start-up, a
 * plug-in running inside someone else's memory-managed runtime, a real-time loop where an
 * allocation would take the driver's global lock.  They still pass A, B, As, Bs and C; what
 * they no longer have to provide is the scratch (status word, split-K tile counters, fp32
 * partial tiles).  That scratch lives in a buffer compiled into the library, of
 * fp8mm_b200_static_scratch_bytes() bytes (8 MiB), which every GPU that loads the library
 * holds until the process exits.
 *
 *   - A (M, N, K, cfg) whose fp8mm_b200_workspace_bytes() exceeds that size is refused with
 *     FP8MM_E_TOO_LARGE before anything is enqueued.  Every unsplit configuration fits.
 *   - The first call on a device looks up the buffer's device address (a synchronous,
 *     non-allocating runtime query, done with that device current).  Make that first call
 *     before starting any stream capture on the device.
 *   - The buffer is shared by all calls and keeps what the last call left in it.  Each call
 *     re-zeroes the tile counters on `stream` before its kernel; the partial tiles are always
 *     written before they are read.  The status word (a bounded device-side wait that gave up)
 *     is left alone, so that it can still be read after later calls:
 *     fp8mm_b200_static_scratch_status().
 *   - Because it is one shared buffer, two calls that can overlap on the GPU (different
 *     streams, or different host threads on different streams) race on it.  Serialise them on
 *     one stream, or use fp8mm_b200_gemm with one workspace per stream.
 *   - Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
 * Results are the same bits fp8mm_b200_gemm produces for the same arguments.
 */
int fp8mm_b200_gemm_static_scratch(const fp8mm_args* args, const fp8mm_cfg* cfg, void* stream);

/* Size in bytes of the built-in scratch buffer used by fp8mm_b200_gemm_static_scratch. */
size_t fp8mm_b200_static_scratch_bytes(void);

/* Status of the calls made through fp8mm_b200_gemm_static_scratch on the current device since
 * the last time this was asked (synchronise the stream first): 0, or FP8MM_E_DEVICE_TIMEOUT with
 * the role/barrier code in *detail (optional); a non-zero status is cleared by reading it.
 * Blocking, allocates nothing.  No counterpart in the reference.  fp8mm_b200_last_status(NULL, ..)
 * reads the same word without clearing it. */
int fp8mm_b200_static_scratch_status(int32_t* detail);

/* Activation quantiser, the step in front of the GEMM: bf16 X[M,K] (row stride ldx) ->
 * e4m3 A[M,K] (contiguous) and fp32 As[M,K/128] (any strides): per 1x128 group
 * scale = max(amax, floor)/448, a = e4m3(clamp(x/scale, +-448)).  Stands where the reference's
 * adapter calls SGLang's sglang_per_token_group_quant_fp8(x, 128, column_major_scales=False,
 * scale_tma_aligned=False) (sgl_patch/fp8mm_sglang_patch.py:53); the recipe is the one of
 * scripts/validate.py:26-28. */
int fp8mm_b200_quantize_act(const void* x_bf16, void* a_e4m3, float* as, int32_t M, int32_t K,
                            int64_t ldx, int64_t as_stride_m, int64_t as_stride_k, float floor_,
                            void* stream);

/* The same with power-of-two scales: the scale of a group is rounded UP to 2^e and written as the
 * UE8M0 byte e + 127 (as_e[M,K/128], strides in bytes), the operand form of FP8MM_IMPL_UMMA_MX.
 * Stands where the adapter calls the same SGLang function with scale_ue8m0=True
 * (sgl_patch/fp8mm_sglang_patch.py:53 with DEEPGEMM_SCALE_UE8M0).  floor_ must be > 0. */
int fp8mm_b200_quantize_act_ue8m0(const void* x_bf16, void* a_e4m3, uint8_t* as_e, int32_t M, int32_t K,
                                  int64_t ldx, int64_t as_stride_m, int64_t as_stride_k, float floor_,
                                  void* stream);

/* UE8M0 scales (8-bit exponent, value 2^(e-127): the scale format of Blackwell block-scaled MMA,
 * which SGLang/DeepGEMM switch to on sm_100) -> contiguous fp32 [rows, kblocks], exactly.
 * packed4 = 0: src is bytes, element (r, kb) at src[r*row_stride + kb*col_stride] (strides in bytes).
 * packed4 = 1: src is int32 words holding four consecutive K blocks each (byte kb%4 of word kb/4,
 *              little endian), word (r, kb/4) at r*row_stride + (kb/4)*col_stride (strides in words),
 *              which covers DeepGEMM's MN-major layout (row_stride 1, col_stride = aligned rows).
 * The reference has no such path: its adapter declines when DEEPGEMM_SCALE_UE8M0 is set
 * (sgl_patch/fp8mm_sglang_patch.py:41), so it never engages on a stock Blackwell SGLang. */
int fp8mm_b200_expand_ue8m0(const void* src, float* dst, int32_t rows, int32_t kblocks,
                            int64_t row_stride, int64_t col_stride, int32_t packed4, void* stream);

/* After the stream has been synchronised: 0 if no bounded device-side wait gave
 * up since the workspace was initialised, else FP8MM_E_DEVICE_TIMEOUT; *detail
 * (optional) receives the role/barrier code recorded by the kernel.  Blocking.
 * workspace == NULL names the built-in scratch of the current device (the one
 * fp8mm_b200_gemm_static_scratch uses). */
int fp8mm_b200_last_status(const void* workspace, int32_t* detail);

/* Text for an error code. */
const char* fp8mm_b200_strerror(int code);

/* Library/ABI version: major*1000 + minor. */
int fp8mm_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FP8MM_B200_H_ */
