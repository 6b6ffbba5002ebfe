// Warp-specialised block-scaled FP8 GEMM for sm_100a.
//
//   C[m,n] = sum_kb ( A[m, 128kb..] . B[n, 128kb..] ) * As[m,kb] * Bs[n/128,kb]      (bf16 out)
//
// One CTA owns one SM and walks a list of work units (output tile x K-split).
// Roles, by warp:
//   warp 0      TMA producer   – streams 128-byte-wide operand tiles into a shared-memory ring
//   warps 1-2   MMA issuers    – per 128-wide K block: four tcgen05.mma (K=32 each) into one of
//                                the TMEM accumulator buffers, fresh accumulator every block;
//                                warp 1 issues the even K blocks, warp 2 the odd ones
//   warp 3      scale loader   – stages the activation/weight scales of the unit in shared memory
//   warps 4..   promotion      – tcgen05.ld the finished K block, acc += d * (As*Bs) in FP32
//                                registers, release the TMEM buffer, finally write bf16 (or the
//                                split-K partial) to global memory
// Promotion of K block k overlaps the MMA of block k+1 through the two TMEM buffers.
//
// The 128 UMMA rows (= TMEM lanes) carry tokens (SWAP=false) or weight rows (SWAP=true, for
// small token counts); the UMMA-N columns carry the other operand.  The math follows the
// reference kernels: fresh accumulator per K block, one scale product per row/column,
// FP32 promote (fp8_gemm_h20/kernels/kernel_v2.py:77-91,164-174), bf16 store or
// fixed-order split-K fix-up through a workspace and a self-resetting counter
// (kernel_v2.py:268-291).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "ptx_sm100.cuh"

namespace fp8mm {

constexpr int kMaxStages = 12;
constexpr int kProducerThreads = 128;  // warps 0-3

// Division of a non-negative 31-bit number by a divisor that is fixed for the launch: one
// multiply-high and a shift (mul = ceil(2^(31+L) / d), L = ceil(log2 d), quotient =
// umulhi(n, mul) >> (L - 1); exact for 0 <= n < 2^31) in place of the ~30 dependent instructions of a
// run-time integer division.  The unit decode has five of them in a row, and it sits on the path
// between two units of a persistent CTA and at the head of a one-unit CTA.
struct FastDiv {
  unsigned int mul, shr, div;
};
inline FastDiv make_fastdiv(int d) {
  FastDiv f;
  f.div = static_cast<unsigned int>(d < 1 ? 1 : d);
  unsigned int L = 0;
  while ((1ull << L) < f.div) ++L;
  if (f.div == 1) { f.mul = 0; f.shr = 0; return f; }
  const unsigned long long pw = 1ull << (31 + L);
  f.mul = static_cast<unsigned int>((pw + f.div - 1) / f.div);
  f.shr = L - 1;
  return f;
}
__host__ __device__ __forceinline__ int fastdiv(int n, const FastDiv& f) {
#ifdef __CUDA_ARCH__
  const unsigned int q = __umulhi(static_cast<unsigned int>(n), f.mul) >> f.shr;
#else
  const unsigned int q = static_cast<unsigned int>((static_cast<unsigned long long>(n) * f.mul) >> 32) >> f.shr;
#endif
  return f.div == 1 ? n : static_cast<int>(q);
}

struct KParams {
  const float* As;
  const float* Bs;
  __nv_bfloat16* C;
  float* ws_partial;   // [tile][split][UMMA_N][128] fp32, split > 1 only
  int* ws_counter;     // [tile], zero between launches
  int* status;         // first word: 0 or the code of the wait that gave up
  long long as_sm, as_sk, bs_sn, bs_sk, ldc;
  unsigned long long timeout_ns;
  int M, N, K;
  int kb_per_unit;     // K blocks per work unit = (K/128)/split
  int split;
  int t_tiles, w_tiles;
  int num_units;       // t_tiles * w_tiles * split
  int group_m;
  FastDiv fd_split, fd_group, fd_gm, fd_tail;   // split, group_m * w_tiles, group_m, size of a ragged last group
  int stages;
  int stg_slabs;       // bf16 staging slabs (32 rows x 64 columns) per epilogue warp: 1 or 2
  int kg;              // K blocks per ring slot (1..8); > 1 only in the KG = 2 kernel variants
  int act_f32;         // block-scaled kernels: As holds float32 powers of two (not exponent bytes)
  long long* trace;    // trace builds only (-DFP8MM_TRACE): clock stamps of CTA 0, else unused
};

// Trace builds record, for 128 consecutive K blocks of CTA 0 (after 64 blocks of warm-up), the SM
// clock at the hand-over points of the three roles: 16 slots per K block.  The product build
// compiles the stamps away.
//   0 producer saw the ring slot empty      1 producer issued the block's copies
//   2 issuer saw the slot full              3 issuer saw the TMEM buffer empty
//   4 issuer issued the block's four MMAs   5 issuer issued both commits
//   6 promotion (first warp) saw the TMEM buffer full      7 its first loads landed
//   8 all its loads landed                  9 it released the buffer     10 it finished the block's FMAs
//  11 promotion (last warp) released the buffer
// and per unit after the CTA's first, in the row of the NEXT unit's first K block (row >= 4):
//  12 epilogue entered   13 tile converted and staged   14 stores handed to the TMA unit
//  15 the next unit's scale table seen
// and in the row after that: 12 staging fenced for the TMA unit   13 warp in step   14 first store
//  issued   15 the next unit's loop entered
// Which waits poll without a suspend hint: bit 0 the promotion warps' wait for a full TMEM buffer,
// bit 1 the MMA issuers' wait for an empty one (the two waits on the loop around a TMEM buffer).
#ifndef FP8MM_SPIN_MASK
#define FP8MM_SPIN_MASK 0
#endif
// Trace builds can also switch parts of the work off (FP8MM_KNOBS: 1 no tcgen05.ld, 2 no operand
// copies, 4 no promotion FMAs) to see what the remaining parts then cost; results are garbage.
#if defined(FP8MM_TRACE) && defined(FP8MM_KNOBS)
#define FP8MM_KNOB(bit_) ((FP8MM_KNOBS & (bit_)) != 0)
#else
#define FP8MM_KNOB(bit_) false
#endif
//  12 kernel entry   13 prologue done (barriers, TMEM, CTA sync)   14 previous grid's results visible
//  15 promotion leader done with the CTA's last unit (its output stored)      (12..15: row 0 only)
// FP8MM_TRACE_FROM (default 64) is the first K block recorded; 0 records a short call from its start.
#ifndef FP8MM_TRACE_FROM
#define FP8MM_TRACE_FROM 64u
#endif
#ifdef FP8MM_TRACE
#define FP8MM_STAMP(slot_, it_)                                                                     \
  do {                                                                                              \
    if (blockIdx.x == 0 && p.trace != nullptr && (it_) >= FP8MM_TRACE_FROM &&                       \
        (it_) < FP8MM_TRACE_FROM + 128u)                                                            \
      p.trace[((it_) - FP8MM_TRACE_FROM) * 16u + (slot_)] = clock64();                              \
  } while (0)
#define FP8MM_STAMP0(slot_)                                                                         \
  do {                                                                                              \
    if (blockIdx.x == 0 && p.trace != nullptr) p.trace[(slot_)] = clock64();                        \
  } while (0)
#else
#define FP8MM_STAMP(slot_, it_) do { } while (0)
#define FP8MM_STAMP0(slot_) do { } while (0)
#endif
// start-up stamps of the roles, in rows 1..3 of the record (slots 12..15 there are otherwise unused):
//  16+12 producer entered   16+13 producer decoded its first unit   16+14 issuer (warp 1) entered
//  16+15 promotion entered  32+12 promotion staged the first unit's scales   32+13 ... saw them complete
//  cluster split-K: 32+14 partial tile parked   32+15 CTA in step   48+12 cluster in step
//                   48+13 this rank's slice reduced and stored (the closing cluster barrier follows)

// Where the bf16 result goes: the caller's C and, for the fused all-gather of the N-sharded
// layer, the same slice of every peer GPU's buffer (plain peer-to-peer stores; the TMA stores
// are ordinary single-destination bulk copies, one per target).
constexpr int kMaxOutTargets = 8;
struct OutTargets {
  CUtensorMap map[kMaxOutTargets];      // token-major tiles: one tensor map per target
  __nv_bfloat16* ptr[kMaxOutTargets];   // swap-AB tiles: plain stores
  int n;
  int pad;
};

struct __align__(8) SharedCtl {
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long tfull[8];    // one per TMEM accumulator buffer
  unsigned long long tempty[8];
  unsigned long long scfull[2];
  unsigned long long scempty[2];
  unsigned int tmem_base;
  int abort;
  int last;
  int pad;
};

// Codes written to the status word when a wait runs out (role * 16 + barrier kind).
enum : int {
  kWaitProducerEmpty = 0x11,
  kWaitMmaFull = 0x21,
  kWaitMmaTmemEmpty = 0x22,
  kWaitLoaderEmpty = 0x31,
  kWaitPromoScale = 0x41,
  kWaitPromoTmemFull = 0x42,
};

struct BoundedWait {
  volatile int* abort;
  int* status;
  unsigned long long limit_ns;
  // Wait for the phase with the given parity.  Gives up after limit_ns (or as soon as
  // another role has given up), records why, and returns false; the caller then leaves
  // its loop so that the CTA can free its TMEM and exit.
  // SPIN: poll without a suspend hint.
  template <bool SPIN = false>
  __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, int code) const {
    auto attempt = [&]() {
      if constexpr (SPIN) return ptx::mbar_try_wait_nohint(bar, parity);
      else return ptx::mbar_try_wait(bar, parity);
    };
    // The slow path is written without a branch out of the polling loop: the loop ends on one
    // condition only, whether the phase completed or the wait gave up.  With a second way out of the
    // loop the register allocator spilled accumulators in the 256-wide kernel's promotion loop
    // (80-120 bytes per thread, 10-13 % of the kernel's time).
    bool done = attempt();
    bool failed = false;
    if (!done) {
      const unsigned long long t0 = ptx::globaltimer_ns();
      do {
        done = attempt();
        const bool stop = (*abort != 0) | (ptx::globaltimer_ns() - t0 > limit_ns);
        failed = stop & !done;
        done |= stop;
      } while (!done);
      if (failed && *abort == 0) {
        *abort = 1;
        if (status != nullptr) atomicCAS(status, 0, code);
      }
    }
    return !failed;
  }
};

struct UnitCoord {
  int tile, ti, wi, s;
};

// Work unit -> (token tile, weight tile, K split).  Tiles are rastered in groups of
// group_m token tiles with the token index fastest, so CTAs that run at the same time
// share weight tiles in L2 (the GROUP_SIZE_M raster of kernel_v2.py:125-134).
__device__ __forceinline__ UnitCoord decode_unit(int u, const KParams& p) {
  UnitCoord c;
  c.tile = fastdiv(u, p.fd_split);
  c.s = u - c.tile * p.split;
  const int g = fastdiv(c.tile, p.fd_group);
  const int first_t = g * p.group_m;
  const int r = c.tile - g * static_cast<int>(p.fd_group.div);
  const bool ragged = first_t + p.group_m > p.t_tiles;   // the last group may hold fewer token tiles
  c.wi = ragged ? fastdiv(r, p.fd_tail) : fastdiv(r, p.fd_gm);
  const int gsz = ragged ? p.t_tiles - first_t : p.group_m;
  c.ti = first_t + r - c.wi * gsz;
  return c;
}

// Stage the scales of one work unit in shared memory: ta[kb][token] = As (times the tile's weight
// scale when SWAP), tb[kb][0..1] = the weight scales of the tile's one or two 128-row blocks
// (token-major tiles only).  Called by NT threads (tid = 0..NT-1).  The table is walked as one flat
// index (kb * TT + token, TT a power of two: no divisions), U independent global loads per thread
// in flight at a time whatever the shape of the table, conflict-free shared-memory stores.
template <int TT, int WT, bool SWAP, int NT, int U>
__device__ __forceinline__ void stage_scales(int tid, const UnitCoord& c, const KParams& p, int kbn,
                                             float* ta, float* tb) {
  static_assert((TT & (TT - 1)) == 0, "token tile must be a power of two");
  const int kb0 = c.s * kbn;
  const int t0 = c.ti * TT;
  const float* as0 = p.As + (long long)kb0 * p.as_sk;
  const float* bs0 = p.Bs + (long long)(c.wi * (WT / 128)) * p.bs_sn + (long long)kb0 * p.bs_sk;
  const int total = kbn * TT;
  // Row-major activation scales (unit stride along K, the layout the quantiser writes): four K
  // blocks of a token per 16-byte load, a quarter of the load instructions and round trips.
  if (p.as_sk == 1 && (p.as_sm & 3) == 0 && ((kb0 | kbn) & 3) == 0 &&
      (reinterpret_cast<unsigned long long>(p.As) & 15ull) == 0) {
    constexpr int UV = U / 4 > 0 ? U / 4 : 1;
    const int quads = (kbn >> 2) * TT;
    for (int base = tid; base < quads; base += NT * UV) {
      float4 v[UV];
#pragma unroll
      for (int u = 0; u < UV; ++u) {
        const int idx = base + u * NT;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (idx < quads) {
          const int kq = idx / TT, x = idx % TT;
          const int tok = min(t0 + x, p.M - 1);
          v[u] = __ldg(reinterpret_cast<const float4*>(as0 + (long long)tok * p.as_sm + kq * 4));
          if (SWAP) {
            const float* b = bs0 + (long long)(kq * 4) * p.bs_sk;
            v[u].x *= __ldg(b);
            v[u].y *= __ldg(b + p.bs_sk);
            v[u].z *= __ldg(b + 2 * p.bs_sk);
            v[u].w *= __ldg(b + 3 * p.bs_sk);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UV; ++u) {
        const int idx = base + u * NT;
        if (idx < quads) {
          const int kq = idx / TT, x = idx % TT;
          float* dst = ta + (kq * 4) * TT + x;
          dst[0] = v[u].x;
          dst[TT] = v[u].y;
          dst[2 * TT] = v[u].z;
          dst[3 * TT] = v[u].w;
        }
      }
    }
  } else
  for (int base = tid; base < total; base += NT * U) {
    float v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int idx = base + u * NT;
      v[u] = 0.f;
      if (idx < total) {
        const int kb = idx / TT, x = idx % TT;
        const int tok = min(t0 + x, p.M - 1);
        v[u] = __ldg(as0 + (long long)tok * p.as_sm + (long long)kb * p.as_sk);
        if (SWAP) v[u] *= __ldg(bs0 + (long long)kb * p.bs_sk);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int idx = base + u * NT;
      if (idx < total) ta[idx] = v[u];
    }
  }
  if (!SWAP) {
    const int nblk_max = p.N / 128 - 1;
    for (int idx = tid; idx < kbn * 2; idx += NT) {
      const int kb = idx >> 1, h = idx & 1;
      const int nb = min(c.wi * (WT / 128) + h, nblk_max);
      tb[idx] = __ldg(p.Bs + (long long)nb * p.bs_sn + (long long)(kb0 + kb) * p.bs_sk);
    }
  }
}

template <int UMMA_N, bool SWAP>
struct KernelTraits {
  static constexpr int NPW = UMMA_N >= 128 ? 8 : 4;           // promotion warps (two column halves when 8)
  static constexpr int CPT = UMMA_N / (NPW / 4);              // accumulator columns per thread
  static constexpr int CH = CPT >= 32 ? 32 : 16;              // columns per tcgen05.ld
  static constexpr int NCH = CPT / CH;
  static constexpr int TT = SWAP ? UMMA_N : 128;              // token tile
  static constexpr int WT = SWAP ? 128 : UMMA_N;              // weight tile
  static constexpr int THREADS = kProducerThreads + NPW * 32;
  static constexpr uint32_t ROW_BYTES = 128u * 128u;
  static constexpr uint32_t COL_BYTES = UMMA_N * 128u;
  static constexpr uint32_t STAGE_BYTES = ROW_BYTES + COL_BYTES;
  // TMEM accumulator buffers, each with its own full/empty barrier pair.  One commit ->
  // promote -> release round trip costs about as much as two 128x256 K blocks of MMA, so the
  // ring should be deep: two buffers is all a 256-column tile can have (512 TMEM columns),
  // 128- and 64-column tiles get four, narrower ones eight.
  static constexpr int NBUF = UMMA_N == 256 ? 2 : (UMMA_N >= 64 ? 4 : 8);
  static constexpr uint32_t TMEM_COLS = NBUF * UMMA_N < 32 ? 32 : NBUF * UMMA_N;
  // bf16 output staging for TMA stores (token-major tiles): 32 rows x 64 columns per warp
  static constexpr uint32_t STAGING_BYTES = SWAP ? 0u : NPW * 4096u;
  static_assert(SWAP || UMMA_N >= 128, "token-major tiles carry 128 or 256 weight rows");
};

// SPLITK: 0 = one CTA owns the whole K range; 1 = fp32 partials through the global workspace;
// 2 = the `split` CTAs of a tile form a thread-block cluster and reduce through distributed
//     shared memory (no workspace, no counters).
// KG = 1: one K block per ring slot.  KG = 2: p.kg (2..8) K blocks per ring slot (small-token tiles,
// K blocks per unit a multiple of p.kg): one 3-D TMA copy per operand brings all of them, which
// divides what the producer thread issues per K block (its ~300 ns per block pace small-token
// calls); the two MMA-issuing threads still alternate over the blocks, so each has at least one
// block in every slot.
template <int UMMA_N, bool SWAP, int SPLITK, int KG = 1>
__global__ void __launch_bounds__(KernelTraits<UMMA_N, SWAP>::THREADS, 1)
fp8mm_umma_kernel(const __grid_constant__ CUtensorMap tm_tok,
                  const __grid_constant__ CUtensorMap tm_wgt,
                  const __grid_constant__ OutTargets outs, const KParams p) {
  using T = KernelTraits<UMMA_N, SWAP>;
  constexpr int NPW = T::NPW, CPT = T::CPT, CH = T::CH, NCH = T::NCH, TT = T::TT, WT = T::WT;
  static_assert(KG == 1 || KG == 2, "one K block per ring slot, or p.kg of them");
  const int kgn = KG == 1 ? 1 : p.kg;
  const uint32_t STAGE_BYTES = T::STAGE_BYTES * (uint32_t)kgn;
  constexpr uint32_t ROW_BYTES = T::ROW_BYTES, COL_BYTES = T::COL_BYTES;
  constexpr int NBUF = T::NBUF;
  constexpr uint32_t IDESC = ptx::idesc_f8_m128(UMMA_N);

  extern __shared__ unsigned char smem_raw[];
  // Operand tiles need 1024-byte alignment for the 128-byte swizzle.
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  unsigned char* smem = smem_raw + pad;
  const uint32_t ring = raw_addr + pad;

  const int kbn = p.kb_per_unit;
  const int stages = p.stages;
  const uint32_t staging = ring + stages * STAGE_BYTES;   // 1024-byte aligned, NPW x slabs x 4 KB
  unsigned char* staging_ptr = smem + (size_t)stages * STAGE_BYTES;
  float* tab_a = reinterpret_cast<float*>(staging_ptr + T::STAGING_BYTES * p.stg_slabs);   // [2][kbn][TT]
  float* tab_b = tab_a + 2 * kbn * TT;                                             // [2][kbn][2]
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(tab_b + 2 * kbn * 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) FP8MM_STAMP0(12);
  // Coordinates of this CTA's first unit, worked out here so that the kernel-parameter fetches and the
  // divisions overlap the barrier set-up and the TMEM allocation below instead of standing between
  // "previous grid done" and the first operand copy (several hundred cycles on every short call).
  // (Not in the 256-column kernels: their promotion loop has no register to spare, and a unit there
  // lasts tens of microseconds.)
  constexpr bool HOIST = UMMA_N < 256;
  UnitCoord c_first = {0, 0, 0, 0};
  if constexpr (HOIST) {
    c_first = decode_unit(blockIdx.x, p);
    asm volatile("" ::"r"(c_first.tile), "r"(c_first.ti), "r"(c_first.wi), "r"(c_first.s));
  }

  const uint32_t bar_full = ptx::smem_u32(&ctl->full[0]);
  const uint32_t bar_empty = ptx::smem_u32(&ctl->empty[0]);
  const uint32_t bar_tfull = ptx::smem_u32(&ctl->tfull[0]);
  const uint32_t bar_tempty = ptx::smem_u32(&ctl->tempty[0]);
  const uint32_t bar_scfull = ptx::smem_u32(&ctl->scfull[0]);
  const uint32_t bar_scempty = ptx::smem_u32(&ctl->scempty[0]);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      // Two arrivals hand a slot back to the producer.  One K block per slot: the commit of the
      // thread that issued its MMAs, and a plain arrive of the other MMA thread once it has seen
      // the slot full (otherwise the slot could be refilled before that thread looked, and its
      // parity wait would be a whole ring pass off).  Two K blocks per slot: both threads' commits.
      ptx::mbar_init(bar_empty + 8 * s, 2);
    }
    for (int b = 0; b < NBUF; ++b) {
      ptx::mbar_init(bar_tfull + 8 * b, 1);
      ptx::mbar_init(bar_tempty + 8 * b, NPW);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_scfull + 8 * b, 32);
      ptx::mbar_init(bar_scempty + 8 * b, NPW);
    }
    ctl->abort = 0;
    ctl->last = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tm_tok);
    ptx::prefetch_tensormap(&tm_wgt);
    if (!SWAP) for (int d = 0; d < outs.n; ++d) ptx::prefetch_tensormap(&outs.map[d]);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&ctl->tmem_base), T::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  if (threadIdx.x == 0) FP8MM_STAMP0(13);

  // Programmatic dependent launch: everything above touched only this CTA's shared memory and
  // TMEM, so it may overlap the tail of the previous kernel in the stream.  From here on
  // global memory is read and written: wait for the previous grid to finish and flush, then
  // let the next grid in the stream start its own prologue early.
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  if (threadIdx.x == 0) FP8MM_STAMP0(14);

  BoundedWait bw{&ctl->abort, p.status, p.timeout_ns};

  // 384-thread variants: the four service warps hand registers to the eight promotion
  // warps, which hold 128 accumulators plus two TMEM load buffers each.  The launch allocates
  // 168 per thread; 128 x (168 - 56) released = 256 x (224 - 168) taken.  At 216 the promotion
  // loop spilled a few values and the packed FMA's register pairs did not fit.
  if (warp < 4) {
  if constexpr (CPT == 128) ptx::setmaxnreg_dec<56>();
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      FP8MM_STAMP0(16 + 12);
      const CUtensorMap* row_map = SWAP ? &tm_wgt : &tm_tok;
      const CUtensorMap* col_map = SWAP ? &tm_tok : &tm_wgt;
      int stage = 0;
      uint32_t ph = 0;
      [[maybe_unused]] uint32_t pit = 0;
      bool first_pass = true;
      bool ok = true;
      for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x) {
        const UnitCoord c = (HOIST && u == (int)blockIdx.x) ? c_first : decode_unit(u, p);
        const int row_y = SWAP ? c.wi * 128 : c.ti * 128;
        const int col_y = SWAP ? c.ti * UMMA_N : c.wi * UMMA_N;
        const int kb0 = c.s * kbn;
        if (pit == 0) FP8MM_STAMP0(16 + 13);
        for (int kb = 0; kb < kbn; kb += kgn) {
          // every slot starts out empty: no wait on the first pass over the ring
          if (!first_pass && !bw.wait(bar_empty + 8 * stage, ph ^ 1u, kWaitProducerEmpty)) { ok = false; break; }
          FP8MM_STAMP(0, pit);
          const uint32_t dst = ring + stage * STAGE_BYTES;
          if (FP8MM_KNOB(2)) {
            ptx::mbar_arrive(bar_full + 8 * stage);
            FP8MM_STAMP(1, pit);
            pit += kgn;
            if (++stage == stages) { stage = 0; ph ^= 1u; first_pass = false; }
            continue;
          }
          ptx::mbar_arrive_expect_tx(bar_full + 8 * stage, STAGE_BYTES);
          if constexpr (KG == 1) {
            ptx::tma_load_2d(dst, row_map, bar_full + 8 * stage, (kb0 + kb) * 128, row_y);
            ptx::tma_load_2d(dst + ROW_BYTES, col_map, bar_full + 8 * stage, (kb0 + kb) * 128, col_y);
          } else {
            // slot layout: [row tile kb] .. [row tile kb+kg-1][column tile kb] .. [column tile kb+kg-1]
            ptx::tma_load_3d(dst, row_map, bar_full + 8 * stage, 0, row_y, kb0 + kb);
            ptx::tma_load_3d(dst + kgn * ROW_BYTES, col_map, bar_full + 8 * stage, 0, col_y, kb0 + kb);
          }
          FP8MM_STAMP(1, pit);
          pit += kgn;
          if (++stage == stages) { stage = 0; ph ^= 1u; first_pass = false; }
        }
      }
    }
    __syncwarp();
  } else if (warp <= 2) {
    // ------------------------------------------------------------- MMA issuers
    // One thread needs ~750 cycles for the waits, the four tcgen05.mma and the commit of a K
    // block, more than the 512 cycles the tensor core needs to run them.  So two threads issue:
    // warp 1 takes the even K blocks (counted over the whole CTA), warp 2 the odd ones.  With an
    // even number of TMEM buffers each thread owns half of them; a tcgen05.commit covers the
    // MMAs of its own thread only, and K blocks are independent (fresh accumulator each).
    if (lane == 0) {
      if (warp == 1) FP8MM_STAMP0(16 + 14);
      const uint32_t par = warp - 1;
      int stage = 0;
      uint32_t ph = 0, it = 0;
      uint32_t jn = 0;              // K block inside the ring slot (always 0 with one block per slot)
      bool ok = true;
      for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x) {
        for (int kb = 0; kb < kbn; ++kb, ++it) {
          const uint32_t j = jn;
          const bool slot_done = KG == 1 || j + 1 == (uint32_t)kgn;
          jn = slot_done ? 0u : j + 1;
          if ((it & 1u) != par) {
            // The other thread's block.  With one K block per slot its operands are still awaited
            // here, so that this thread sees every slot of the ring fill in order: a parity wait
            // can only tell the current phase from the one before, and a slot whose previous fill
            // this thread had never seen complete could otherwise read as "already full".  (With
            // several blocks per slot each thread owns at least one block of every slot and waits
            // on all.)
            if constexpr (KG == 1) {
              if (!bw.wait(bar_full + 8 * stage, ph, kWaitMmaFull)) { ok = false; break; }
              ptx::mbar_arrive(bar_empty + 8 * stage);     // seen: the slot may be refilled
            }
            if (slot_done && ++stage == stages) { stage = 0; ph ^= 1u; }
            continue;
          }
          const uint32_t buf = it % NBUF, tph = (it / NBUF) & 1u;
          if (!bw.wait(bar_full + 8 * stage, ph, kWaitMmaFull)) { ok = false; break; }
          FP8MM_STAMP(2, it);
          const uint32_t a_addr = ring + stage * STAGE_BYTES + j * ROW_BYTES;
          const uint64_t a_desc = ptx::smem_desc_k128(a_addr);
          if (!bw.wait<(FP8MM_SPIN_MASK & 2) != 0>(bar_tempty + 8 * buf, tph ^ 1u, kWaitMmaTmemEmpty)) { ok = false; break; }
          FP8MM_STAMP(3, it);
          ptx::tc_fence_after();
          const uint64_t b_desc = ptx::smem_desc_k128(ring + stage * STAGE_BYTES + kgn * ROW_BYTES + j * COL_BYTES);
          const uint32_t d_tmem = tmem_base + buf * UMMA_N;
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k) {
            // 32 fp8 = 32 bytes along K inside the swizzle span: +2 in 16-byte address units.
            ptx::umma_f8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, k);
          }
          FP8MM_STAMP(4, it);
          ptx::umma_commit(bar_tfull + 8 * buf);   // this K block's partial product is ready
          // A second commit hands the K block's operand tiles back to the producer once these MMAs
          // have retired.  (A commit covers the MMAs of its own thread, i.e. exactly this block.)
          // With two issuing threads there is time for it here, and it takes one barrier operation
          // per K block off the promotion warps, whose pace every other role follows.
          // (Several blocks per slot: the last two blocks of a slot belong to the two threads, and
          // each thread's commit after its last block covers its earlier blocks of the slot too.)
          if (KG == 1 || j + 2 >= (uint32_t)kgn) ptx::umma_commit(bar_empty + 8 * stage);
          FP8MM_STAMP(5, it);
          if (slot_done && ++stage == stages) { stage = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ scale loader
    // Prefetches the scale tables of the CTA's second and later units while the previous unit is
    // being promoted.  The first unit's tables are staged by the promotion warps themselves (they
    // have nothing else to do until the first MMAs retire, and they are 4-8x as many threads);
    // for that unit this warp only arrives, which keeps the barrier phases in step.
    const int tid = threadIdx.x - 96;     // warp 3
    uint32_t ui = 0;
    for (int u = blockIdx.x; u < p.num_units; u += gridDim.x, ++ui) {
      const UnitCoord c = (HOIST && ui == 0) ? c_first : decode_unit(u, p);
      const uint32_t t = ui & 1u, tph = (ui >> 1) & 1u;
      if (!bw.wait(bar_scempty + 8 * t, tph ^ 1u, kWaitLoaderEmpty)) break;
      if (ui > 0) stage_scales<TT, WT, SWAP, 32, 16>(tid, c, p, kbn, tab_a + t * kbn * TT, tab_b + t * kbn * 2);
      ptx::mbar_arrive(bar_scfull + 8 * t);
    }
  }
  } else {
    // ------------------------------------------------- promotion + epilogue warps
    if constexpr (CPT == 128) ptx::setmaxnreg_inc<224>();
    const int pw = warp - 4;
    const int q = warp & 3;      // TMEM lane quarter this warp may read
    const int half = pw >> 2;    // which 128-column half of a 256-wide tile
    const int row = q * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + half * CPT;
    const bool leader = threadIdx.x == kProducerThreads;
    if (leader) FP8MM_STAMP0(16 + 15);
    uint32_t ui = 0, it = 0;
    for (int u = blockIdx.x; u < p.num_units; u += gridDim.x, ++ui) {
      const UnitCoord c = (HOIST && ui == 0) ? c_first : decode_unit(u, p);
      if (leader && ui > 0 && it >= 4) FP8MM_STAMP(15, it + 1);
      const uint32_t t = ui & 1u, sph = (ui >> 1) & 1u;
      if (ui == 0) {
        // first unit of the CTA: all promotion threads stage its scales (one round of loads)
        stage_scales<TT, WT, SWAP, NPW * 32, 8>(threadIdx.x - kProducerThreads, c, p, kbn, tab_a, tab_b);
        ptx::bar_sync(1, NPW * 32);
        if (leader) FP8MM_STAMP0(32 + 12);
      }
      bool ok = bw.wait(bar_scfull + 8 * t, sph, kWaitPromoScale);
      if (leader && ui == 0) FP8MM_STAMP0(32 + 13);
      if (leader && ui > 0 && it >= 4) FP8MM_STAMP(15, it);
      const float* ta = tab_a + t * kbn * TT;
      const float* tb = tab_b + t * kbn * 2;

      float acc[CPT];
#pragma unroll
      for (int j = 0; j < CPT; ++j) acc[j] = 0.f;

      for (int kb = 0; kb < kbn && ok; ++kb, ++it) {
        const uint32_t buf = it % NBUF, tph = (it / NBUF) & 1u;
        float sc = 0.f;
        if (!SWAP) sc = ta[kb * TT + row] * tb[kb * 2 + (half * CPT) / 128];
        const float4* sv = reinterpret_cast<const float4*>(ta + kb * TT + half * CPT);
        const uint32_t tb_idx = buf;
        if (!bw.wait<(FP8MM_SPIN_MASK & 1) != 0>(bar_tfull + 8 * tb_idx, tph, kWaitPromoTmemFull)) { ok = false; break; }
        [[maybe_unused]] const bool tr_first = leader;
        [[maybe_unused]] const bool tr_last = threadIdx.x == kProducerThreads + (NPW - 1) * 32;
        if (tr_first) FP8MM_STAMP(6, it);
        ptx::tc_fence_after();
        const uint32_t taddr = lane_base + buf * UMMA_N;
// One pair of accumulator columns: the packed FP32 FMA takes half the issue slots of two fmaf and
// gives the same bits.  The promotion warps share their SM sub-partition's issue port with one
// another and with the service warps, and their FMAs were half of all instructions issued.
#define FP8MM_PROMOTE_CHUNK_(FMA_, dd_, ch_)                                                       \
  do {                                                                                             \
    if (SWAP) {                                                                                    \
      _Pragma("unroll") for (int i_ = 0; i_ < CH; i_ += 4) {                                       \
        const float4 s4_ = sv[((ch_) * CH + i_) >> 2];                                             \
        FMA_(acc[(ch_) * CH + i_], acc[(ch_) * CH + i_ + 1], dd_[i_], dd_[i_ + 1], s4_.x, s4_.y);  \
        FMA_(acc[(ch_) * CH + i_ + 2], acc[(ch_) * CH + i_ + 3], dd_[i_ + 2], dd_[i_ + 3], s4_.z,  \
             s4_.w);                                                                               \
      }                                                                                            \
    } else {                                                                                       \
      _Pragma("unroll") for (int i_ = 0; i_ < CH; i_ += 2)                                         \
        FMA_(acc[(ch_) * CH + i_], acc[(ch_) * CH + i_ + 1], dd_[i_], dd_[i_ + 1], sc, sc);        \
    }                                                                                              \
  } while (0)
#define FP8MM_PROMOTE_CHUNK(dd_, ch_)                                                              \
  do {                                                                                             \
    if (FP8MM_KNOB(4)) break;                                                                      \
    FP8MM_PROMOTE_CHUNK_(ptx::ffma2, dd_, ch_);                                                    \
  } while (0)
        uint32_t d[2][CH];
        if constexpr (NCH <= 2) {
          // up to 64 columns per thread: every load in flight at once, one wait, then release
          // the buffer before any FMA
          if (!FP8MM_KNOB(1)) ptx::tmem_ld<CH>(taddr, d[0]);
          if constexpr (NCH == 2) ptx::tmem_ld<CH>(taddr + CH, d[1]);
          ptx::tmem_wait_ld();
          if (tr_first) FP8MM_STAMP(8, it);
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar_tempty + 8 * tb_idx);
          if (tr_first) FP8MM_STAMP(9, it);
          if (tr_last) FP8MM_STAMP(11, it);
          FP8MM_PROMOTE_CHUNK(d[0], 0);
          if constexpr (NCH == 2) FP8MM_PROMOTE_CHUNK(d[1], 1);
          if (tr_first) FP8MM_STAMP(10, it);
        } else {
          // 128 columns per thread in two waits instead of four: the chain from "MMAs done" to
          // "buffer handed back" is two TMEM round trips plus 32 FMAs, and it is that chain (with
          // only two 256-column buffers) that paces the kernel, not the FMA or load throughput.
          static_assert(NCH == 4, "two pairs of 32-column loads");
          if (!FP8MM_KNOB(1)) ptx::tmem_ld<CH>(taddr, d[0]);
          if (!FP8MM_KNOB(1)) ptx::tmem_ld<CH>(taddr + CH, d[1]);
          ptx::tmem_wait_ld();
          if (tr_first) FP8MM_STAMP(7, it);
          FP8MM_PROMOTE_CHUNK(d[0], 0);
          if (!FP8MM_KNOB(1)) ptx::tmem_ld<CH>(taddr + 2 * CH, d[0]);
          FP8MM_PROMOTE_CHUNK(d[1], 1);
          if (!FP8MM_KNOB(1)) ptx::tmem_ld<CH>(taddr + 3 * CH, d[1]);
          ptx::tmem_wait_ld();
          if (tr_first) FP8MM_STAMP(8, it);
          // every tcgen05.ld of this warp has completed: hand the buffer back before the last
          // FMAs so the next MMA into it can be issued as early as possible
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar_tempty + 8 * tb_idx);
          if (tr_first) FP8MM_STAMP(9, it);
          if (tr_last) FP8MM_STAMP(11, it);
          FP8MM_PROMOTE_CHUNK(d[0], 2);
          FP8MM_PROMOTE_CHUNK(d[1], 3);
          if (tr_first) FP8MM_STAMP(10, it);
        }
#undef FP8MM_PROMOTE_CHUNK
#undef FP8MM_PROMOTE_CHUNK_
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar_scempty + 8 * t);

      // ------------------------------------------------------------- epilogue
      if (leader && it >= 4) FP8MM_STAMP(12, it);
      if constexpr (SPLITK == 2) {
        // Cluster split-K: park the fp32 partial in this CTA's own shared memory (the operand ring
        // is idle: this CTA's only unit is finished); the reduction follows the cluster barrier.
        // Swap-AB tiles park column-major ([token column][128 weight rows], the output's order);
        // token-major tiles park row-major with rows padded by four floats, so that the 16-byte
        // stores here and the 16-byte loads of the reduction are free of bank conflicts.
        if (ok) {
          if constexpr (SWAP) {
            float* red = reinterpret_cast<float*>(smem) + (size_t)(half * CPT) * 128 + row;
#pragma unroll
            for (int j = 0; j < CPT; ++j) red[j * 128] = acc[j];
          } else {
            float4* red = reinterpret_cast<float4*>(reinterpret_cast<float*>(smem) +
                                                    (size_t)row * (UMMA_N + 4) + half * CPT);
#pragma unroll
            for (int j = 0; j < CPT; j += 4) red[j >> 2] = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
          }
        }
        break;
      } else if constexpr (SPLITK == 1) {
        // Split-K: park the fp32 partial; the CTA that arrives last on the tile's counter
        // sums all partials in split order (bit-stable) and writes the tile.
        const size_t tile_floats = (size_t)UMMA_N * 128;
        float* part = p.ws_partial + ((size_t)c.tile * p.split + c.s) * tile_floats +
                      (size_t)(half * CPT) * 128 + row;
        if (ok) {
#pragma unroll
          for (int j = 0; j < CPT; ++j) __stcg(part + j * 128, acc[j]);
        }
        __threadfence();
        ptx::bar_sync(1, NPW * 32);
        if (leader) {
          int verdict = 2;  // 2 = a wait gave up somewhere in this CTA: stop
          if (!ctl->abort) {
            const int old = atomicAdd(p.ws_counter + c.tile, 1);
            verdict = (old == p.split - 1) ? 1 : 0;
          }
          ctl->last = verdict;
        }
        ptx::bar_sync(1, NPW * 32);
        const int verdict = ctl->last;
        if (verdict == 2) break;
        if (verdict == 0) continue;
        __threadfence();
        const float* base = p.ws_partial + (size_t)c.tile * p.split * tile_floats +
                            (size_t)(half * CPT) * 128 + row;
        if constexpr (CPT <= 32) {
          // narrow tiles: the loads of up to 64/CPT splits are in flight together (one L2 round
          // trip instead of one per split); the additions still run in split order
          constexpr int SG = 64 / CPT;
          for (int s0 = 0; s0 < p.split; s0 += SG) {
            float v[SG][CPT];
#pragma unroll
            for (int ss = 0; ss < SG; ++ss) {
              if (s0 + ss < p.split) {
#pragma unroll
                for (int j = 0; j < CPT; ++j) v[ss][j] = __ldcg(base + (size_t)(s0 + ss) * tile_floats + j * 128);
              }
            }
#pragma unroll
            for (int ss = 0; ss < SG; ++ss) {
              if (s0 + ss < p.split) {
#pragma unroll
                for (int j = 0; j < CPT; ++j) acc[j] = (s0 + ss == 0) ? v[ss][j] : acc[j] + v[ss][j];
              }
            }
          }
        } else {
          constexpr int RB = CPT == 64 ? 32 : 16;   // loads per batch
          for (int s = 0; s < p.split; ++s) {
            const float* src = base + s * tile_floats;
#pragma unroll
            for (int j0 = 0; j0 < CPT; j0 += RB) {
              float v[RB];
#pragma unroll
              for (int i = 0; i < RB; ++i) v[i] = __ldcg(src + (size_t)(j0 + i) * 128);
#pragma unroll
              for (int i = 0; i < RB; ++i) acc[j0 + i] = (s == 0) ? v[i] : acc[j0 + i] + v[i];
              asm volatile("" ::: "memory");  // bound the loads in flight per thread (registers)
            }
          }
        }
        if (leader) atomicExch(p.ws_counter + c.tile, 0);
      } else {
        if (!ok) break;
      }

      if (SWAP) {
        const int n = c.wi * 128 + row;
        const int m_base = c.ti * TT + half * CPT;
        const int m_left = p.M - m_base;
        for (int d = 0; d < outs.n; ++d) {
          __nv_bfloat16* dst = outs.ptr[d] + (long long)m_base * p.ldc + n;
#pragma unroll
          for (int j = 0; j < CPT; ++j) {
            if (j < m_left) *dst = __float2bfloat16_rn(acc[j]);
            dst += p.ldc;
          }
        }
      } else {
        // Coalesced bf16 epilogue: each warp stages its 32 rows x 64 columns in shared memory
        // (128-byte rows, 16-byte chunks XOR-swizzled by row so the writes are conflict-free)
        // and one lane hands the slab to the TMA unit, which clips it at the edges of C.
        const int m0w = c.ti * 128 + q * 32;
        const int n0 = c.wi * WT + half * CPT;
        if (m0w < p.M && n0 < p.N) {
          // With two slabs per warp (256-wide tiles, when shared memory allows) both halves of the
          // warp's 128 columns are staged back to back and lanes 0 and 1 issue one store each; the
          // wait for the TMA unit to have read the staging memory then falls at the start of the
          // NEXT unit's epilogue, a whole main loop later, instead of between the two slabs.
          const int nsl = p.stg_slabs;
          unsigned char* stg = staging_ptr + pw * 4096 * nsl;
          const uint32_t stg_addr = staging + pw * 4096 * nsl;
          constexpr int SLABS = CPT >= 64 ? CPT / 64 : 1;
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) {
            const int so = (nsl == 2) ? sl * 4096 : 0;
            if (sl == 0 || nsl == 1) {
              if (lane < 2 * kMaxOutTargets) ptx::bulk_wait_read_all();   // earlier slabs have left the staging buffer
              __syncwarp();
            }
#pragma unroll
            for (int ck = 0; ck < 8; ++ck) {
              const int j = sl * 64 + ck * 8;
              __nv_bfloat162 v0 = __floats2bfloat162_rn(acc[j + 0], acc[j + 1]);
              __nv_bfloat162 v1 = __floats2bfloat162_rn(acc[j + 2], acc[j + 3]);
              __nv_bfloat162 v2 = __floats2bfloat162_rn(acc[j + 4], acc[j + 5]);
              __nv_bfloat162 v3 = __floats2bfloat162_rn(acc[j + 6], acc[j + 7]);
              uint4 o;
              o.x = *reinterpret_cast<uint32_t*>(&v0);
              o.y = *reinterpret_cast<uint32_t*>(&v1);
              o.z = *reinterpret_cast<uint32_t*>(&v2);
              o.w = *reinterpret_cast<uint32_t*>(&v3);
              *reinterpret_cast<uint4*>(stg + so + lane * 128 + ((ck ^ (lane & 7)) << 4)) = o;
            }
            // One issuing lane per (target, slab): a thread pays a few hundred cycles per TMA
            // instruction, and with up to eight targets (fused all-gather) a single lane would
            // spend longer issuing the stores than the tile took to compute.
            if (leader && sl == SLABS - 1 && it >= 4) FP8MM_STAMP(13, it);
            if (nsl == 1) {
              ptx::fence_proxy_async_smem();
              __syncwarp();
              if (lane < outs.n) {
                ptx::tma_store_2d(&outs.map[lane], stg_addr, n0 + sl * 64, m0w);
                ptx::bulk_commit_group();
              }
            } else if (sl == SLABS - 1) {
              ptx::fence_proxy_async_smem();
              if (leader && it >= 4) FP8MM_STAMP(12, it + 1);
              __syncwarp();
              if (leader && it >= 4) FP8MM_STAMP(13, it + 1);
              if (lane < SLABS * outs.n) {
                const int d = lane / SLABS, ls = lane % SLABS;
                ptx::tma_store_2d(&outs.map[d], stg_addr + ls * 4096, n0 + ls * 64, m0w);
                if (leader && it >= 4) FP8MM_STAMP(14, it + 1);
                ptx::bulk_commit_group();
              }
            }
            if (leader && sl == SLABS - 1 && it >= 4) FP8MM_STAMP(14, it);
          }
        }
      }
    }
    if (!SWAP && lane < 2 * kMaxOutTargets) ptx::bulk_wait_all();   // stores (also those to peer GPUs) are done
    __syncwarp();
  }

  if constexpr (SPLITK == 2) {
    // ------------------------------------------------- cluster split-K reduction
    // Rank r of the cluster reduces the r-th slice of the tile (token columns of a swap-AB tile,
    // token rows of a token-major one) over all ranks in rank order (the same order as the
    // workspace path: bit-identical results) and writes that slice of the output.
    if (threadIdx.x == kProducerThreads) FP8MM_STAMP0(32 + 14);    // partial tile parked
    __syncthreads();
    if (threadIdx.x == kProducerThreads) FP8MM_STAMP0(32 + 15);    // CTA in step
    ptx::cluster_sync_all();             // every CTA's partial tile is in its shared memory
    if (threadIdx.x == kProducerThreads) FP8MM_STAMP0(48 + 12);    // cluster in step
    if (warp >= 4 && blockIdx.x < p.num_units) {
      const UnitCoord c = HOIST ? c_first : decode_unit(blockIdx.x, p);
      const int pw = warp - 4;
      // A rank whose bounded wait gave up has parked nothing: then no rank stores the tile.  The
      // flags travel with the first batch of partial-tile loads (same round trip) and are looked
      // at only where the stores are issued.
      uint32_t bad = 0;
      {
        const uint32_t abort_addr = ptx::smem_u32(&ctl->abort);
#pragma unroll
        for (int s = 0; s < 8; ++s)
          if (s < p.split) bad |= ptx::ld_cluster_u32(ptx::map_to_cta(abort_addr, s));
      }
      if (SWAP) {
        // The partial tiles lie column-major ([token column][128 weight rows]), and any rank may
        // reduce any column as long as the additions run in rank order.  Rank r takes the columns
        // [r, r+1) * UMMA_N / split; a warp takes whole columns, a lane four consecutive weight
        // rows: one 16-byte distributed-shared-memory load per rank and column (a quarter of the
        // requests of scalar loads, all ranks of two columns in flight together) and one 8-byte
        // store of four bf16, 256 contiguous bytes per warp.
        const int cpr = UMMA_N / p.split;
        const int col0 = (int)ptx::cluster_ctarank() * cpr;
        const uint32_t rbase = ring + (uint32_t)(4 * lane) * 4u;
        const int n = c.wi * 128 + 4 * lane;
        for (int i = pw; i < cpr; i += 2 * NPW) {
          float4 x[2][8];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
#pragma unroll
            for (int s = 0; s < 8; ++s) {
              x[u][s] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (s < p.split && i + u * NPW < cpr)
                x[u][s] = ptx::ld_cluster_f32x4(ptx::map_to_cta(rbase + (uint32_t)(col0 + i + u * NPW) * 512u, s));
            }
          }
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            float4 v = x[u][0];
#pragma unroll
            for (int s = 1; s < 8; ++s) {
              if (s < p.split) {
                v.x += x[u][s].x;
                v.y += x[u][s].y;
                v.z += x[u][s].z;
                v.w += x[u][s].w;
              }
            }
            const int m = c.ti * TT + col0 + i + u * NPW;
            if (i + u * NPW < cpr && m < p.M && bad == 0) {
              __nv_bfloat162 b0 = __floats2bfloat162_rn(v.x, v.y), b1 = __floats2bfloat162_rn(v.z, v.w);
              uint2 o;
              o.x = *reinterpret_cast<uint32_t*>(&b0);
              o.y = *reinterpret_cast<uint32_t*>(&b1);
              for (int d = 0; d < outs.n; ++d)
                *reinterpret_cast<uint2*>(outs.ptr[d] + (long long)m * p.ldc + n) = o;
            }
          }
        }
      } else {
        // Token-major tiles: rank r reduces the rows [r, r+1) * 128 / split; a warp takes whole rows,
        // a lane four consecutive weight columns of each 128-column block: one 16-byte load per
        // rank (all ranks of a row in flight together) and 8-byte stores, 256 contiguous bytes per
        // warp.  The additions run in rank order, as on the workspace path.
        const int rpr = 128 / p.split;
        const int row0 = (int)ptx::cluster_ctarank() * rpr;
        for (int i = pw; i < rpr; i += NPW) {
          const int r = row0 + i;
          const int m = c.ti * 128 + r;
#pragma unroll
          for (int cb = 0; cb < UMMA_N / 128; ++cb) {
            const int col = cb * 128 + 4 * lane;
            const uint32_t addr = ring + ((uint32_t)r * (UMMA_N + 4) + (uint32_t)col) * 4u;
            float4 x[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) {
              x[s] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (s < p.split) x[s] = ptx::ld_cluster_f32x4(ptx::map_to_cta(addr, s));
            }
            float4 v = x[0];
#pragma unroll
            for (int s = 1; s < 8; ++s) {
              if (s < p.split) {
                v.x += x[s].x;
                v.y += x[s].y;
                v.z += x[s].z;
                v.w += x[s].w;
              }
            }
            const int n = c.wi * WT + col;
            if (m < p.M && n < p.N && bad == 0) {
              __nv_bfloat162 b0 = __floats2bfloat162_rn(v.x, v.y), b1 = __floats2bfloat162_rn(v.z, v.w);
              uint2 o;
              o.x = *reinterpret_cast<uint32_t*>(&b0);
              o.y = *reinterpret_cast<uint32_t*>(&b1);
              for (int d = 0; d < outs.n; ++d)
                *reinterpret_cast<uint2*>(outs.ptr[d] + (long long)m * p.ldc + n) = o;
            }
          }
        }
      }
    }
    if (threadIdx.x == kProducerThreads) FP8MM_STAMP0(48 + 13);    // this rank's slice reduced and stored
    ptx::cluster_sync_all();             // no rank reads this CTA's shared memory any more
  }

  // ---------------------------------------------------------------- teardown
  if (threadIdx.x == kProducerThreads) FP8MM_STAMP0(15);
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (ctl->abort) __nanosleep(1000000);  // let copies that are still in flight land
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}

}  // namespace fp8mm
