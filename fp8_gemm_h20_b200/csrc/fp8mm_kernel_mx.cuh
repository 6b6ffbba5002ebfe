// Block-scaled FP8 GEMM for power-of-two (UE8M0) scales on the tensor cores' own scaling path.
//
//   C[M,N] (bf16) = sum_kb 2^(As[m,kb]-127) * 2^(Bs[n/128,kb]-127) * (A[m, kb] . B[n, kb])
//
// with As, Bs given as UE8M0 bytes (the exponent alone), the form DeepSeek-style checkpoints use on
// Blackwell.  `tcgen05.mma.kind::mxf8f6f4.block_scale` multiplies every 32-deep slice of the dot
// product by one scale per row of A and one per row of B, read from tensor memory, and accumulates in
// FP32 in tensor memory over the whole K: no per-K-block trip of the accumulators through registers
// (the promotion that paces fp8mm_umma_kernel), one accumulator drain per tile.
//
// The reference has one scale per 128 of K (kernel_v2.py:77-91); the instruction wants one per 32.
// The scale operand is a 32-bit word per row holding four bytes, and the instruction descriptor's
// scale-factor ids pick the byte: so a word holds the scales of FOUR CONSECUTIVE K BLOCKS, and all
// four MMAs of K block kb use byte kb % 4.  Per four K blocks the scales of a tile are one 512-byte
// atom for the 128 token rows and two for the 256 weight rows ([32 lanes][4 words]: word c of lane l
// belongs to row 32 c + l), copied shared memory -> tensor memory by `tcgen05.cp.32x128b.warpx4`.
//
// One CTA per SM, 128 x 256 tiles, persistent.  Warps: 0 TMA producer, 1 MMA issuer (one thread: all
// MMAs of a tile go to the same accumulator), 2 scale loader, 3 idle, 4-11 epilogue (tcgen05.ld of the
// finished accumulator, bf16, swizzled staging, TMA store).  Tensor memory: columns 0-255 the
// accumulator, 256-287 two slots of scale words.  The accumulator is handed back to the issuer as soon
// as every epilogue warp has it in registers.
#pragma once
#include "fp8mm_kernel.cuh"

namespace fp8mm {
namespace ptx {

__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}
// 32 rows x 16 bytes of shared memory -> 32 lanes x 4 columns of tensor memory, repeated in all four
// lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// Shared-memory descriptor of one scale atom: 32 rows of 16 bytes back to back = four 8-row core
// matrices 128 bytes apart, no swizzle.
__device__ __forceinline__ uint64_t smem_desc_sf(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(16 >> 4) << 16;     // leading byte offset (one 16-byte column only)
  d |= static_cast<uint64_t>(128 >> 4) << 32;    // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;           // descriptor version of sm_100
  return d;
}
// Instruction descriptor of the block-scaled form: e4m3 x e4m3, K-major, UE8M0 scales, M = 128;
// `sf` = which byte of the scale words both operands use.
__host__ __device__ constexpr uint32_t idesc_mxf8_m128(uint32_t n, uint32_t sf) {
  return (sf << 4)               // B scale-factor id
         | (0u << 7)             // A format e4m3
         | (0u << 10)            // B format e4m3
         | ((n >> 3) << 17)      // N / 8
         | (1u << 23)            // scale format E8M0
         | ((128u >> 4) << 24)   // M / 16
         | (sf << 29);           // A scale-factor id
}

}  // namespace ptx

// UE8M0 byte of the activation scale at element `at`: read as a byte, or taken from the exponent field
// of a float32 power of two (what a quantiser with power-of-two scales hands over as floats).
__device__ __forceinline__ uint32_t mx_act_scale(const KParams& p, long long at) {
  if (p.act_f32) return (__float_as_uint(__ldg(p.As + at)) >> 23) & 0xFFu;
  return static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned char*>(p.As) + at));
}

struct __align__(8) MxCtl {
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long sffull[2];
  unsigned long long sfempty[2];
  unsigned long long accfull;
  unsigned long long accempty;
  unsigned int tmem_base;
  int abort;
  int last;      // split-K: verdict of the tile's counter for this CTA's epilogue warps
  int reserved;
};

// Codes of the waits of this kernel (role * 16 + barrier kind), next to those of fp8mm_umma_kernel.
enum : int {
  kWaitMxIssuerScales = 0x23,
  kWaitMxIssuerAcc = 0x24,
  kWaitMxLoaderEmpty = 0x33,
  kWaitMxEpilogueAcc = 0x44,
};

struct MxTraits {
  static constexpr int UMMA_N = 256;
  static constexpr int THREADS = kProducerThreads + 8 * 32;
  static constexpr uint32_t ROW_BYTES = 128u * 128u;      // 128 token rows of one K block
  static constexpr uint32_t COL_BYTES = 256u * 128u;      // 256 weight rows
  static constexpr uint32_t STAGE_BYTES = ROW_BYTES + COL_BYTES;
  static constexpr uint32_t STAGING_BYTES = 8u * 2u * 4096u;
  static constexpr uint32_t SF_SLOT_BYTES = 3u * 512u;    // tokens, weight rows 0-127, weight rows 128-255
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t SF_COL = 256;                 // first scale column; 16 columns per slot
};

__global__ void __launch_bounds__(MxTraits::THREADS, 1)
fp8mm_mx_kernel(const __grid_constant__ CUtensorMap tm_tok, const __grid_constant__ CUtensorMap tm_wgt,
                const __grid_constant__ OutTargets outs, const KParams p) {
  using T = MxTraits;
  constexpr uint32_t STAGE_BYTES = T::STAGE_BYTES;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  unsigned char* smem = smem_raw + pad;
  const uint32_t ring = raw_addr + pad;

  const int kbn = p.kb_per_unit;
  const int stages = p.stages;
  const uint32_t staging = ring + stages * STAGE_BYTES;
  unsigned char* staging_ptr = smem + (size_t)stages * STAGE_BYTES;
  const uint32_t sf_smem = staging + T::STAGING_BYTES;
  MxCtl* ctl = reinterpret_cast<MxCtl*>(staging_ptr + T::STAGING_BYTES + 2 * T::SF_SLOT_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t bar_full = ptx::smem_u32(&ctl->full[0]);
  const uint32_t bar_empty = ptx::smem_u32(&ctl->empty[0]);
  const uint32_t bar_sffull = ptx::smem_u32(&ctl->sffull[0]);
  const uint32_t bar_sfempty = ptx::smem_u32(&ctl->sfempty[0]);
  const uint32_t bar_accfull = ptx::smem_u32(&ctl->accfull);
  const uint32_t bar_accempty = ptx::smem_u32(&ctl->accempty);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(bar_sffull + 8 * s, 32);
      ptx::mbar_init(bar_sfempty + 8 * s, 1);
    }
    ptx::mbar_init(bar_accfull, 1);
    ptx::mbar_init(bar_accempty, 8);
    ctl->abort = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tm_tok);
    ptx::prefetch_tensormap(&tm_wgt);
    for (int d = 0; d < outs.n; ++d) ptx::prefetch_tensormap(&outs.map[d]);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&ctl->tmem_base), T::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();

  BoundedWait bw{&ctl->abort, p.status, p.timeout_ns};
  const unsigned char* As8 = reinterpret_cast<const unsigned char*>(p.As);
  const unsigned char* Bs8 = reinterpret_cast<const unsigned char*>(p.Bs);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t ph = 0;
      bool first_pass = true, ok = true;
      for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x) {
        const UnitCoord c = decode_unit(u, p);
        for (int kb = 0; kb < kbn; ++kb) {
          if (!first_pass && !bw.wait(bar_empty + 8 * stage, ph ^ 1u, kWaitProducerEmpty)) { ok = false; break; }
          const uint32_t dst = ring + stage * STAGE_BYTES;
          ptx::mbar_arrive_expect_tx(bar_full + 8 * stage, STAGE_BYTES);
          ptx::tma_load_2d(dst, &tm_tok, bar_full + 8 * stage, kb * 128, c.ti * 128);
          ptx::tma_load_2d(dst + T::ROW_BYTES, &tm_wgt, bar_full + 8 * stage, kb * 128, c.wi * 256);
          if (++stage == stages) { stage = 0; ph ^= 1u; first_pass = false; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t ph = 0, ui = 0, gi = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x, ++ui) {
        // the epilogue warps hold the previous tile in registers: the accumulator may be overwritten
        if (ui > 0 && !bw.wait(bar_accempty, (ui - 1) & 1u, kWaitMxIssuerAcc)) break;
        ptx::tc_fence_after();
        for (int kb = 0; kb < kbn; ++kb) {
          const uint32_t slot = gi & 1u;
          const uint32_t tsf = tmem_base + T::SF_COL + slot * 16u;
          if ((kb & 3) == 0) {
            if (!bw.wait(bar_sffull + 8 * slot, (gi >> 1) & 1u, kWaitMxIssuerScales)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint32_t src = sf_smem + slot * T::SF_SLOT_BYTES;
            ptx::tmem_cp_32x128b_warpx4(tsf, ptx::smem_desc_sf(src));
            ptx::tmem_cp_32x128b_warpx4(tsf + 8u, ptx::smem_desc_sf(src + 512u));
            ptx::tmem_cp_32x128b_warpx4(tsf + 12u, ptx::smem_desc_sf(src + 1024u));
          }
          if (!bw.wait(bar_full + 8 * stage, ph, kWaitMmaFull)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_addr = ring + stage * STAGE_BYTES;
          const uint64_t a_desc = ptx::smem_desc_k128(a_addr);
          const uint64_t b_desc = ptx::smem_desc_k128(a_addr + T::ROW_BYTES);
          const uint32_t idesc = ptx::idesc_mxf8_m128(T::UMMA_N, static_cast<uint32_t>(kb & 3));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            ptx::umma_mxf8(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, tsf, tsf + 8u,
                           static_cast<uint32_t>((kb | k) != 0));
          ptx::umma_commit(bar_empty + 8 * stage);
          if ((kb & 3) == 3 || kb == kbn - 1) {
            ptx::umma_commit(bar_sfempty + 8 * slot);   // scale words and their shared-memory atoms are free
            ++gi;
          }
          if (++stage == stages) { stage = 0; ph ^= 1u; }
        }
        if (ok) ptx::umma_commit(bar_accfull);
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------ scale loader
    // Per four K blocks: the UE8M0 bytes of the tile's 128 token rows and 2 weight-row blocks, packed
    // four K blocks to a word, in the [32 lanes][4 words] order the copy to tensor memory expects.
    uint32_t gi = 0;
    bool ok = true;
    const int nblk_max = p.N / 128 - 1;
    for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x) {
      const UnitCoord c = decode_unit(u, p);
      for (int kb0 = 0; kb0 < kbn; kb0 += 4, ++gi) {
        const uint32_t slot = gi & 1u, use = gi >> 1;
        if (use > 0 && !bw.wait(bar_sfempty + 8 * slot, (use - 1) & 1u, kWaitMxLoaderEmpty)) { ok = false; break; }
        uint32_t wa[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int tok = min(c.ti * 128 + q * 32 + lane, p.M - 1);
          const long long at = (long long)tok * p.as_sm + (long long)kb0 * p.as_sk;
          uint32_t w = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t b = (kb0 + j < kbn) ? mx_act_scale(p, at + (long long)j * p.as_sk) : 127u;
            w |= b << (8 * j);
          }
          wa[q] = w;
        }
        uint32_t wb[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int nb = min(c.wi * 2 + h, nblk_max);
          const unsigned char* src = Bs8 + (long long)nb * p.bs_sn + (long long)kb0 * p.bs_sk;
          uint32_t w = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t b = (kb0 + j < kbn) ? static_cast<uint32_t>(__ldg(src + (long long)j * p.bs_sk)) : 127u;
            w |= b << (8 * j);
          }
          wb[h] = w;
        }
        const uint32_t dst = sf_smem + slot * T::SF_SLOT_BYTES + lane * 16u;
        ptx::sts_v4(dst, wa[0], wa[1], wa[2], wa[3]);
        ptx::sts_v4(dst + 512u, wb[0], wb[0], wb[0], wb[0]);
        ptx::sts_v4(dst + 1024u, wb[1], wb[1], wb[1], wb[1]);
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive(bar_sffull + 8 * slot);
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------- epilogue warps
    const int pw = warp - 4;
    const int q = warp & 3;      // TMEM lane quarter this warp may read
    const int half = pw >> 2;    // which 128 columns of the tile
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + half * 128;
    unsigned char* stg = staging_ptr + pw * 8192;
    const uint32_t stg_addr = staging + pw * 8192;
    uint32_t ui = 0;
    for (int u = blockIdx.x; u < p.num_units; u += gridDim.x, ++ui) {
      const UnitCoord c = decode_unit(u, p);
      if (!bw.wait(bar_accfull, ui & 1u, kWaitMxEpilogueAcc)) break;
      ptx::tc_fence_after();
      uint32_t d[4][32];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) ptx::tmem_ld<32>(taddr + ch * 32, d[ch]);
      ptx::tmem_wait_ld();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar_accempty);
      const int m0w = c.ti * 128 + q * 32;
      const int n0 = c.wi * 256 + half * 128;
      if (m0w < p.M && n0 < p.N) {
        if (lane < 2 * kMaxOutTargets) ptx::bulk_wait_read_all();   // the previous tile has left the staging memory
        __syncwarp();
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
#pragma unroll
          for (int ck = 0; ck < 8; ++ck) {
            const uint32_t* v = &d[sl * 2 + (ck >> 2)][(ck & 3) * 8];
            __nv_bfloat162 v0 = __floats2bfloat162_rn(__uint_as_float(v[0]), __uint_as_float(v[1]));
            __nv_bfloat162 v1 = __floats2bfloat162_rn(__uint_as_float(v[2]), __uint_as_float(v[3]));
            __nv_bfloat162 v2 = __floats2bfloat162_rn(__uint_as_float(v[4]), __uint_as_float(v[5]));
            __nv_bfloat162 v3 = __floats2bfloat162_rn(__uint_as_float(v[6]), __uint_as_float(v[7]));
            uint4 o;
            o.x = *reinterpret_cast<uint32_t*>(&v0);
            o.y = *reinterpret_cast<uint32_t*>(&v1);
            o.z = *reinterpret_cast<uint32_t*>(&v2);
            o.w = *reinterpret_cast<uint32_t*>(&v3);
            *reinterpret_cast<uint4*>(stg + sl * 4096 + lane * 128 + ((ck ^ (lane & 7)) << 4)) = o;
          }
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane < 2 * outs.n) {
          const int dd = lane >> 1, ls = lane & 1;
          ptx::tma_store_2d(&outs.map[dd], stg_addr + ls * 4096, n0 + ls * 64, m0w);
          ptx::bulk_commit_group();
        }
      }
    }
    if (lane < 2 * kMaxOutTargets) ptx::bulk_wait_all();
    __syncwarp();
  }

  // teardown: every role is out of its loop (or has given up); free the tensor memory
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (ctl->abort) __nanosleep(1000000);  // let copies that are still in flight land
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}


// ---------------------------------------------------------------------------------------------
// The same with 256 x 224 tiles: two 128-row accumulators side by side in tensor memory
// (2 x 224 columns, the scale words in the 64 that remain), each fed by its own MMA-issuing thread
// from the SAME weight tile in shared memory.  A 128 x 256 tile draws 48 KB of operands per K block
// through an L2-to-SM path that delivers ~65 bytes per clock, i.e. ~790 cycles for 512 cycles of MMA;
// this tile draws 60 KB for 896 cycles of MMA, so the tensor pipe, not the delivery, sets the pace.
// Epilogue warps take all 224 columns of their rows into registers as packed bf16 (112 registers),
// hand the accumulator back, and then stage and store 32-column pieces while the next tile runs.
struct Mx256Traits {
  static constexpr int UMMA_N = 224;
  static constexpr int THREADS = kProducerThreads + 8 * 32;
  static constexpr uint32_t ROW_BYTES = 256u * 128u;      // 256 token rows of one K block
  static constexpr uint32_t COL_BYTES = 224u * 128u;      // 224 weight rows
  static constexpr uint32_t STAGE_BYTES = ROW_BYTES + COL_BYTES;
  static constexpr uint32_t STAGING_BYTES = 8u * 2u * 2048u;   // two 32 x 32 bf16 slabs per epilogue warp
  static constexpr uint32_t SF_SLOT_BYTES = 4u * 512u;    // token rows 0-127, 128-255, weight rows 0-127, 128-223
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t SF_COL = 448;                 // 24 columns per slot: per issuer 4 (tokens) + 8 (weights)
};

__global__ void __launch_bounds__(Mx256Traits::THREADS, 1)
fp8mm_mx256_kernel(const __grid_constant__ CUtensorMap tm_tok, const __grid_constant__ CUtensorMap tm_wgt,
                   const __grid_constant__ OutTargets outs, const KParams p) {
  using T = Mx256Traits;
  constexpr uint32_t STAGE_BYTES = T::STAGE_BYTES;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  unsigned char* smem = smem_raw + pad;
  const uint32_t ring = raw_addr + pad;

  const int kbn = p.kb_per_unit;
  const int stages = p.stages;
  const uint32_t staging = ring + stages * STAGE_BYTES;
  unsigned char* staging_ptr = smem + (size_t)stages * STAGE_BYTES;
  const uint32_t sf_smem = staging + T::STAGING_BYTES;
  MxCtl* ctl = reinterpret_cast<MxCtl*>(staging_ptr + T::STAGING_BYTES + 2 * T::SF_SLOT_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t bar_full = ptx::smem_u32(&ctl->full[0]);
  const uint32_t bar_empty = ptx::smem_u32(&ctl->empty[0]);
  const uint32_t bar_sffull = ptx::smem_u32(&ctl->sffull[0]);
  const uint32_t bar_sfempty = ptx::smem_u32(&ctl->sfempty[0]);
  const uint32_t bar_accfull = ptx::smem_u32(&ctl->accfull);
  const uint32_t bar_accempty = ptx::smem_u32(&ctl->accempty);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 2);     // the commits of both issuing threads
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(bar_sffull + 8 * s, 32);
      ptx::mbar_init(bar_sfempty + 8 * s, 2);
    }
    ptx::mbar_init(bar_accfull, 2);
    ptx::mbar_init(bar_accempty, 8);
    ctl->abort = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tm_tok);
    ptx::prefetch_tensormap(&tm_wgt);
    for (int d = 0; d < outs.n; ++d) ptx::prefetch_tensormap(&outs.map[d]);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&ctl->tmem_base), T::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();

  BoundedWait bw{&ctl->abort, p.status, p.timeout_ns};
  const unsigned char* As8 = reinterpret_cast<const unsigned char*>(p.As);
  const unsigned char* Bs8 = reinterpret_cast<const unsigned char*>(p.Bs);

  if (warp < 4) {
  ptx::setmaxnreg_dec<56>();
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t ph = 0;
      bool first_pass = true, ok = true;
      for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x) {
        const UnitCoord c = decode_unit(u, p);
        for (int kb = 0; kb < kbn; ++kb) {
          if (!first_pass && !bw.wait(bar_empty + 8 * stage, ph ^ 1u, kWaitProducerEmpty)) { ok = false; break; }
          const uint32_t dst = ring + stage * STAGE_BYTES;
          ptx::mbar_arrive_expect_tx(bar_full + 8 * stage, STAGE_BYTES);
          ptx::tma_load_2d(dst, &tm_tok, bar_full + 8 * stage, kb * 128, c.ti * 256);
          ptx::tma_load_2d(dst + T::ROW_BYTES, &tm_wgt, bar_full + 8 * stage, kb * 128, c.wi * T::UMMA_N);
          if (++stage == stages) { stage = 0; ph ^= 1u; first_pass = false; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1 || warp == 3) {
    // ------------------------------------------------------------- MMA issuers
    // Warp 1 owns the accumulator of token rows 0-127, warp 3 that of rows 128-255; they share nothing
    // but the operand ring (each copies the scale words it needs into its own tensor-memory columns).
    if (lane == 0) {
      const uint32_t h = warp == 1 ? 0u : 1u;
      const uint32_t d_tmem = tmem_base + h * T::UMMA_N;
      int stage = 0;
      uint32_t ph = 0, ui = 0, gi = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x, ++ui) {
        if (ui > 0 && !bw.wait(bar_accempty, (ui - 1) & 1u, kWaitMxIssuerAcc)) break;
        ptx::tc_fence_after();
        for (int kb = 0; kb < kbn; ++kb) {
          const uint32_t slot = gi & 1u;
          const uint32_t tsf = tmem_base + T::SF_COL + slot * 24u + h * 12u;
          if ((kb & 3) == 0) {
            if (!bw.wait(bar_sffull + 8 * slot, (gi >> 1) & 1u, kWaitMxIssuerScales)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint32_t src = sf_smem + slot * T::SF_SLOT_BYTES;
            ptx::tmem_cp_32x128b_warpx4(tsf, ptx::smem_desc_sf(src + h * 512u));
            ptx::tmem_cp_32x128b_warpx4(tsf + 4u, ptx::smem_desc_sf(src + 1024u));
            ptx::tmem_cp_32x128b_warpx4(tsf + 8u, ptx::smem_desc_sf(src + 1536u));
          }
          if (!bw.wait(bar_full + 8 * stage, ph, kWaitMmaFull)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_addr = ring + stage * STAGE_BYTES;
          const uint64_t a_desc = ptx::smem_desc_k128(a_addr + h * (128u * 128u));
          const uint64_t b_desc = ptx::smem_desc_k128(a_addr + T::ROW_BYTES);
          const uint32_t idesc = ptx::idesc_mxf8_m128(T::UMMA_N, static_cast<uint32_t>(kb & 3));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            ptx::umma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, tsf, tsf + 4u,
                           static_cast<uint32_t>((kb | k) != 0));
          ptx::umma_commit(bar_empty + 8 * stage);
          if ((kb & 3) == 3 || kb == kbn - 1) {
            ptx::umma_commit(bar_sfempty + 8 * slot);
            ++gi;
          }
          if (++stage == stages) { stage = 0; ph ^= 1u; }
        }
        if (ok) ptx::umma_commit(bar_accfull);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ scale loader
    // Per four K blocks four atoms: token rows 0-127 and 128-255, weight rows 0-127 and 128-223 of the
    // tile (a 224-row weight tile does not start on a 128-row scale block: the block of every row is
    // worked out by itself).
    uint32_t gi = 0;
    bool ok = true;
    const int nblk_max = p.N / 128 - 1;
    const bool quick_a = !p.act_f32 && p.as_sk == 1 && (p.as_sm & 3) == 0 && (reinterpret_cast<unsigned long long>(As8) & 3ull) == 0;
    for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x) {
      const UnitCoord c = decode_unit(u, p);
      for (int kb0 = 0; kb0 < kbn; kb0 += 4, ++gi) {
        const uint32_t slot = gi & 1u, use = gi >> 1;
        if (use > 0 && !bw.wait(bar_sfempty + 8 * slot, (use - 1) & 1u, kWaitMxLoaderEmpty)) { ok = false; break; }
        const bool whole = kb0 + 3 < kbn;
        uint32_t w[16];
#pragma unroll
        for (int q = 0; q < 8; ++q) {        // token rows q * 32 + lane
          const int tok = min(c.ti * 256 + q * 32 + lane, p.M - 1);
          const long long at = (long long)tok * p.as_sm + (long long)kb0 * p.as_sk;
          uint32_t v = 0;
          if (quick_a && whole) {
            v = __ldg(reinterpret_cast<const uint32_t*>(As8 + at));
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              v |= ((kb0 + j < kbn) ? mx_act_scale(p, at + (long long)j * p.as_sk) : 127u) << (8 * j);
          }
          w[q] = v;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {        // weight rows q * 32 + lane of the tile (those past 223 are unused)
          const int nb = min((c.wi * T::UMMA_N + q * 32 + lane) >> 7, nblk_max);
          const unsigned char* src = Bs8 + (long long)nb * p.bs_sn + (long long)kb0 * p.bs_sk;
          uint32_t v = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            v |= ((kb0 + j < kbn) ? static_cast<uint32_t>(__ldg(src + (long long)j * p.bs_sk)) : 127u) << (8 * j);
          w[8 + q] = v;
        }
        const uint32_t dst = sf_smem + slot * T::SF_SLOT_BYTES + lane * 16u;
#pragma unroll
        for (int a = 0; a < 4; ++a) ptx::sts_v4(dst + a * 512u, w[4 * a], w[4 * a + 1], w[4 * a + 2], w[4 * a + 3]);
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive(bar_sffull + 8 * slot);
      }
    }
  }
  } else {
    // ---------------------------------------------------------- epilogue warps
    ptx::setmaxnreg_inc<224>();
    const int pw = warp - 4;
    const int q = warp & 3;      // TMEM lane quarter this warp may read
    const int h = pw >> 2;       // which accumulator (token rows 0-127 or 128-255 of the tile)
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + h * T::UMMA_N;
    unsigned char* stg = staging_ptr + pw * 4096;
    const uint32_t stg_addr = staging + pw * 4096;
    uint32_t ui = 0, pieces = 0;   // pieces staged so far: consecutive pieces alternate between the two slabs
    for (int u = blockIdx.x; u < p.num_units; u += gridDim.x, ++ui) {
      const UnitCoord c = decode_unit(u, p);
      if (!bw.wait(bar_accfull, ui & 1u, kWaitMxEpilogueAcc)) break;
      ptx::tc_fence_after();
      uint32_t pk[112];          // the thread's 224 columns as bf16 pairs
      {
        uint32_t d[4][32];
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) ptx::tmem_ld<32>(taddr + ch * 32, d[ch]);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(d[ch][i]), __uint_as_float(d[ch][i + 1]));
            pk[ch * 16 + (i >> 1)] = *reinterpret_cast<uint32_t*>(&v);
          }
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) ptx::tmem_ld<32>(taddr + 128 + ch * 32, d[ch]);
        ptx::tmem_wait_ld();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_accempty);     // the accumulator may be overwritten
#pragma unroll
        for (int ch = 0; ch < 3; ++ch)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(d[ch][i]), __uint_as_float(d[ch][i + 1]));
            pk[64 + ch * 16 + (i >> 1)] = *reinterpret_cast<uint32_t*>(&v);
          }
      }
      const int m0w = c.ti * 256 + h * 128 + q * 32;
      const int n0 = c.wi * T::UMMA_N;
      if (m0w < p.M) {
        // seven pieces of 32 columns through two 2 KB slabs (64-byte rows, 16-byte chunks XOR-swizzled
        // by row pair = the TMA unit's 64-byte swizzle); a slab is rewritten once the store issued
        // two pieces earlier has read it
#pragma unroll
        for (int pc = 0; pc < 7; ++pc, ++pieces) {
          if (n0 + pc * 32 >= p.N) break;      // past the edge of C: only stored pieces take turns on the slabs
          if (lane < kMaxOutTargets) ptx::bulk_wait_read_1();
          __syncwarp();
          const uint32_t so = (pieces & 1u) * 2048u;
          unsigned char* slab = stg + so;
#pragma unroll
          for (int ck = 0; ck < 4; ++ck) {
            uint4 o = make_uint4(pk[pc * 16 + ck * 4], pk[pc * 16 + ck * 4 + 1], pk[pc * 16 + ck * 4 + 2],
                                 pk[pc * 16 + ck * 4 + 3]);
            *reinterpret_cast<uint4*>(slab + lane * 64 + ((ck ^ ((lane >> 1) & 3)) << 4)) = o;
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane < outs.n) {
            ptx::tma_store_2d(&outs.map[lane], stg_addr + so, n0 + pc * 32, m0w);
            ptx::bulk_commit_group();
          }
        }
      }
    }
    if (lane < kMaxOutTargets) ptx::bulk_wait_all();
    __syncwarp();
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (ctl->abort) __nanosleep(1000000);  // let copies that are still in flight land
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}


// ---------------------------------------------------------------------------------------------
// Small token counts with power-of-two scales: swap-AB tiles of 128 weight rows (on the 128 rows of
// the MMA) x TT tokens (on its N), the whole K accumulated in tensor memory.  Nothing crosses registers
// per K block (the table kernels promote every block).  What paces such a CTA is the ISSUE
// of the MMAs: ~90 cycles per tcgen05.mma for its thread, four per K block, whatever the tile's width.
// So NI threads in NI warps issue, thread i the K blocks kb % NI == i, each into its OWN accumulator
// (TT columns) and from its OWN copy of the scale words; the epilogue adds the NI accumulators in
// issuer order.  A ring slot holds NI K blocks, fetched by ONE 3-D copy per operand (the producing
// thread pays per copy too): thread i takes block i of every slot; blocks of the last slot past the unit's K range are not used.  Scale words: one atom for the weight rows (one scale block: every word the same), one
// for the tokens.  Four epilogue warps read the accumulators 32 columns at a time and store bf16 with
// plain stores (a thread owns a weight row = a column of C).
// Split-K (layers with too few weight tiles for the SMs): units of (tile, K split).  With a split of 2, 4 or
// 8 the CTAs of a tile form a cluster, park their fp32 partials in their own shared memory and rank r adds
// the r-th slice of token columns over distributed shared memory; otherwise every unit parks its partial in
// the workspace and the last one to arrive on the tile's counter adds them.  Both add in split order.
// Warps: 0 producer, 1 scale loader, 2..5 MMA issuers (2..3 for 128 tokens), 6..9 epilogue.
// The half-size form (NI_ = 2 on tiles of up to 64 tokens): half the ring slot and half the tensor memory, so
// that two CTAs share an SM (each with its own issuing threads; one CTA's prologue and epilogue run under the
// other's main loop).  Measured with 64-token tiles where the units outnumber the SMs: 9.8 us against 11.6 at
// 256 x 9216 x 2048, 15.3 against 19.1 at 1024 x 2048 x 4096.  (A one-issuer form of the 128-token tile was tried
// too: ~990 cycles per K block, no better than the two-issuer tile.)
template <int TT, int NI_ = (TT <= 64 ? 4 : 2)>
struct MxsTraits {
  static_assert(TT == 16 || TT == 32 || TT == 64 || TT == 128, "token tile");
  static_assert((NI_ == 4 && TT <= 64) || NI_ == 2, "issuing threads");
  static constexpr int NI = NI_;                              // issuing threads = accumulators
  static constexpr int SERVICE = 6 * 32;
  static constexpr int THREADS = SERVICE + 4 * 32;
  static constexpr uint32_t ROW_BYTES = 128u * 128u;          // 128 weight rows of one K block
  static constexpr uint32_t COL_BYTES = (uint32_t)TT * 128u;  // TT tokens
  static constexpr uint32_t STAGE_BYTES = NI * (ROW_BYTES + COL_BYTES);   // NI K blocks per slot
  static constexpr uint32_t SF_SLOT_BYTES = 2u * 512u;
  static constexpr uint32_t SF_COL = (uint32_t)(NI * TT);     // per issuer and slot 8 columns
  static constexpr uint32_t USED_COLS = SF_COL + NI * 16u;
  static constexpr uint32_t TMEM_COLS = USED_COLS <= 32 ? 32u : (USED_COLS <= 64 ? 64u : (USED_COLS <= 128 ? 128u : (USED_COLS <= 256 ? 256u : 512u)));
};

// Split-K tail of fp8mm_mxs_kernel: add the fp32 partials of one tile in split order and write bf16.  Called by
// the four epilogue warps of the CTA that arrived last on the tile's counter; kept out of line so that the
// common path's registers do not pay for it.
template <int TT>
__device__ __noinline__ void mxs_reduce_tile(const float* base, int split, int M, long long ldc,
                                             const OutTargets& outs, int m_base, int n) {
  const size_t tile_floats = (size_t)TT * 128;
  constexpr int RC = 16;             // token columns per pass
  constexpr int SG = 4;              // splits whose loads are in flight together (one L2 round trip)
#pragma unroll 1
  for (int c0 = 0; c0 < TT; c0 += RC) {
    if (m_base + c0 >= M) break;
    float acc[RC];
    for (int s0 = 0; s0 < split; s0 += SG) {
      float v[SG][RC];
#pragma unroll
      for (int ss = 0; ss < SG; ++ss) {
        if (s0 + ss < split) {
          const float* src = base + (size_t)(s0 + ss) * tile_floats + (size_t)c0 * 128;
#pragma unroll
          for (int j = 0; j < RC; ++j) v[ss][j] = __ldcg(src + (size_t)j * 128);
        }
      }
#pragma unroll
      for (int ss = 0; ss < SG; ++ss) {
        if (s0 + ss < split) {
#pragma unroll
          for (int j = 0; j < RC; ++j) acc[j] = (s0 + ss == 0) ? v[ss][j] : acc[j] + v[ss][j];
        }
      }
    }
    const int m_left = M - (m_base + c0);
    for (int t = 0; t < outs.n; ++t) {
      __nv_bfloat16* dst = outs.ptr[t] + (long long)(m_base + c0) * ldc + n;
#pragma unroll
      for (int j = 0; j < RC; ++j) {
        if (j < m_left) *dst = __float2bfloat16_rn(acc[j]);
        dst += ldc;
      }
    }
  }
}

// Cluster split-K tail of fp8mm_mxs_kernel: the partials lie [token column][128 weight rows]; this rank owns
// the token columns [rank, rank + 1) * TT / S, warp pw of the four epilogue warps every fourth of them, a lane
// four consecutive weight rows: 16-byte loads from the S ranks' shared memory, up to 16 in flight per lane (a
// load from another SM takes about a microsecond), added in rank order, 8-byte stores (256 contiguous bytes per warp).
template <int TT, int S>
__device__ __forceinline__ void mxs_reduce_cols(uint32_t ring, int pw, int lane, const UnitCoord& c, const KParams& p,
                                                const OutTargets& outs, uint32_t bad) {
  constexpr int CPR = TT / S;                     // this rank's columns
  constexpr int CPW = (CPR + 3) / 4;              // per warp
  constexpr int BATCH = CPW * S <= 16 ? CPW : 16 / S;
  const uint32_t my_rank = ptx::cluster_ctarank();
  const int col0 = (int)my_rank * CPR;
  const uint32_t rbase = ring + (uint32_t)lane * 16u;
  const int n = c.wi * 128 + 4 * lane;
#pragma unroll
  for (int c0 = 0; c0 < CPW; c0 += BATCH) {
    float4 x[BATCH][S];
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const int cl = pw + 4 * (c0 + i);
#pragma unroll
      for (int s = 0; s < S; ++s) {
        x[i][s] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (cl < CPR) x[i][s] = ptx::ld_rank_f32x4(rbase + (uint32_t)(col0 + cl) * 512u, s, my_rank);
      }
    }
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const int cl = pw + 4 * (c0 + i);
      float4 v = x[i][0];
#pragma unroll
      for (int s = 1; s < S; ++s) {
        v.x += x[i][s].x;
        v.y += x[i][s].y;
        v.z += x[i][s].z;
        v.w += x[i][s].w;
      }
      const int m = c.ti * TT + col0 + cl;
      if (cl < CPR && m < p.M && bad == 0) {
        __nv_bfloat162 b0 = __floats2bfloat162_rn(v.x, v.y), b1 = __floats2bfloat162_rn(v.z, v.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&b0);
        o.y = *reinterpret_cast<uint32_t*>(&b1);
        for (int t = 0; t < outs.n; ++t)
          *reinterpret_cast<uint2*>(outs.ptr[t] + (long long)m * p.ldc + n) = o;
      }
    }
  }
}

// SPLITK: 0 = one unit per tile, 1 = split-K through the workspace, 2 = through a cluster.
template <int TT, int SPLITK = 0, int NI_ = (TT <= 64 ? 4 : 2)>
__global__ void __launch_bounds__(MxsTraits<TT, NI_>::THREADS, 1)
fp8mm_mxs_kernel(const __grid_constant__ CUtensorMap tm_tok, const __grid_constant__ CUtensorMap tm_wgt,
                 const __grid_constant__ OutTargets outs, const KParams p) {
  using T = MxsTraits<TT, NI_>;
  constexpr uint32_t STAGE_BYTES = T::STAGE_BYTES;
  constexpr int NI = T::NI;
  constexpr bool kSplit = SPLITK != 0;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  unsigned char* smem = smem_raw + pad;
  const uint32_t ring = raw_addr + pad;

  const int kbn = p.kb_per_unit;
  const int stages = p.stages;
  const uint32_t sf_smem = ring + stages * STAGE_BYTES;
  MxCtl* ctl = reinterpret_cast<MxCtl*>(smem + (size_t)stages * STAGE_BYTES + 2 * T::SF_SLOT_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t bar_full = ptx::smem_u32(&ctl->full[0]);
  const uint32_t bar_empty = ptx::smem_u32(&ctl->empty[0]);
  const uint32_t bar_sffull = ptx::smem_u32(&ctl->sffull[0]);
  const uint32_t bar_sfempty = ptx::smem_u32(&ctl->sfempty[0]);
  const uint32_t bar_accfull = ptx::smem_u32(&ctl->accfull);
  const uint32_t bar_accempty = ptx::smem_u32(&ctl->accempty);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, NI);       // every issuing thread's commit: each takes one block of the slot
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(bar_sffull + 8 * s, 32);
      ptx::mbar_init(bar_sfempty + 8 * s, NI);
    }
    ptx::mbar_init(bar_accfull, NI);
    ptx::mbar_init(bar_accempty, 4);
    ctl->abort = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tm_tok);
    ptx::prefetch_tensormap(&tm_wgt);
  }
  if (warp == 2) {
    ptx::tmem_alloc(ptx::smem_u32(&ctl->tmem_base), T::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();

  BoundedWait bw{&ctl->abort, p.status, p.timeout_ns};
  const unsigned char* As8 = reinterpret_cast<const unsigned char*>(p.As);
  const unsigned char* Bs8 = reinterpret_cast<const unsigned char*>(p.Bs);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t ph = 0;
      bool first_pass = true, ok = true;
      for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x) {
        const UnitCoord c = decode_unit(u, p);
        const int kbo = kSplit ? c.s * kbn : 0;    // this split's first K block
        for (int kb = 0; kb < kbn; kb += NI) {
          if (!first_pass && !bw.wait(bar_empty + 8 * stage, ph ^ 1u, kWaitProducerEmpty)) { ok = false; break; }
          const uint32_t dst = ring + stage * STAGE_BYTES;
          ptx::mbar_arrive_expect_tx(bar_full + 8 * stage, STAGE_BYTES);
          // slot layout: [weight tile kb] .. [weight tile kb+NI-1][token tile kb] .. [token tile kb+NI-1]
          ptx::tma_load_3d(dst, &tm_wgt, bar_full + 8 * stage, 0, c.wi * 128, kbo + kb);
          ptx::tma_load_3d(dst + NI * T::ROW_BYTES, &tm_tok, bar_full + 8 * stage, 0, c.ti * TT, kbo + kb);
          if (++stage == stages) { stage = 0; ph ^= 1u; first_pass = false; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ scale loader
    uint32_t gi = 0;
    bool ok = true;
    const int nblk_max = p.N / 128 - 1;
    for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x) {
      const UnitCoord c = decode_unit(u, p);
      const int kbo = kSplit ? c.s * kbn : 0;
      for (int kb0 = 0; kb0 < kbn; kb0 += 4, ++gi) {
        const uint32_t slot = gi & 1u, use = gi >> 1;
        if (use > 0 && !bw.wait(bar_sfempty + 8 * slot, (use - 1) & 1u, kWaitMxLoaderEmpty)) { ok = false; break; }
        uint32_t wt[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          wt[q] = 0x7F7F7F7Fu;
          if (q * 32 < TT) {
            const int tok = min(c.ti * TT + q * 32 + lane, p.M - 1);
            const long long at = (long long)tok * p.as_sm + (long long)(kbo + kb0) * p.as_sk;
            uint32_t v = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              v |= ((kb0 + j < kbn) ? mx_act_scale(p, at + (long long)j * p.as_sk) : 127u) << (8 * j);
            wt[q] = v;
          }
        }
        const unsigned char* srcw = Bs8 + (long long)min(c.wi, nblk_max) * p.bs_sn + (long long)(kbo + kb0) * p.bs_sk;
        uint32_t ww = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          ww |= ((kb0 + j < kbn) ? static_cast<uint32_t>(__ldg(srcw + (long long)j * p.bs_sk)) : 127u) << (8 * j);
        const uint32_t dst = sf_smem + slot * T::SF_SLOT_BYTES + lane * 16u;
        ptx::sts_v4(dst, ww, ww, ww, ww);
        ptx::sts_v4(dst + 512u, wt[0], wt[1], wt[2], wt[3]);
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive(bar_sffull + 8 * slot);
      }
    }
  } else if (warp < 2 + NI) {
    // ------------------------------------------------------------- MMA issuers
    if (lane == 0) {
      const uint32_t id = warp - 2;
      const uint32_t d_tmem = tmem_base + id * TT;
      int stage = 0;
      uint32_t ph = 0, ui = 0, gi = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x, ++ui) {
        if (ui > 0 && !bw.wait(bar_accempty, (ui - 1) & 1u, kWaitMxIssuerAcc)) break;
        ptx::tc_fence_after();
        bool first = true;         // this thread's first MMA of the unit overwrites its accumulator
        for (int kb0 = 0; kb0 < kbn; kb0 += NI) {
          const int kb = kb0 + (int)id;                       // this thread's block of the slot
          const uint32_t slot = gi & 1u;
          const uint32_t tsf = tmem_base + T::SF_COL + id * 16u + slot * 8u;
          if ((kb0 & 3) == 0) {
            if (!bw.wait(bar_sffull + 8 * slot, (gi >> 1) & 1u, kWaitMxIssuerScales)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint32_t src = sf_smem + slot * T::SF_SLOT_BYTES;
            ptx::tmem_cp_32x128b_warpx4(tsf, ptx::smem_desc_sf(src));
            ptx::tmem_cp_32x128b_warpx4(tsf + 4u, ptx::smem_desc_sf(src + 512u));
          }
          if (!bw.wait(bar_full + 8 * stage, ph, kWaitMmaFull)) { ok = false; break; }
          ptx::tc_fence_after();
          // the last slot of a split's K range reaches into the next split's blocks: not used.  (Unsplit, the
          // blocks past K arrive as zeros, the copy's out-of-bounds fill, and add nothing.)
          if (!kSplit || kb < kbn) {
            const uint32_t base = ring + stage * STAGE_BYTES;
            const uint64_t a_desc = ptx::smem_desc_k128(base + id * T::ROW_BYTES);
            const uint64_t b_desc = ptx::smem_desc_k128(base + NI * T::ROW_BYTES + id * T::COL_BYTES);
            const uint32_t idesc = ptx::idesc_mxf8_m128(TT, static_cast<uint32_t>(kb & 3));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              ptx::umma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, tsf, tsf + 4u,
                             static_cast<uint32_t>(!(first && k == 0)));
            first = false;
          }
          ptx::umma_commit(bar_empty + 8 * stage);
          if (((kb0 + NI) & 3) == 0 || kb0 + NI >= kbn) {
            ptx::umma_commit(bar_sfempty + 8 * slot);   // this thread's MMAs and copies of the group are done
            ++gi;
          }
          if (++stage == stages) { stage = 0; ph ^= 1u; }
        }
        if (ok) ptx::umma_commit(bar_accfull);
      }
    }
    __syncwarp();
  } else if (warp >= 6) {
    // ---------------------------------------------------------- epilogue warps
    const int q = warp & 3;
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    constexpr int CH = TT >= 32 ? 32 : 16;
    const int n_acc = (kSplit && kbn < NI) ? kbn : NI;     // issuing threads that had a K block in this unit
    const bool leader = threadIdx.x == T::SERVICE;
    const size_t tile_floats = (size_t)TT * 128;
    uint32_t ui = 0;
    for (int u = blockIdx.x; u < p.num_units; u += gridDim.x, ++ui) {
      const UnitCoord c = decode_unit(u, p);
      const int row = q * 32 + lane;
      const int n = c.wi * 128 + row;
      const int m_base = c.ti * TT;
      // split-K: this unit's fp32 partial goes to the workspace, [token column][128 weight rows]
      float* part = SPLITK == 1 ? p.ws_partial + ((size_t)c.tile * p.split + c.s) * tile_floats + row : nullptr;
      const bool ok = bw.wait(bar_accfull, ui & 1u, kWaitMxEpilogueAcc);
      if (!ok && part == nullptr) break;
      // (with split-K a warp whose wait gave up still meets the other three at the barrier below, where
      // the leader sees the abort flag and all four leave together)
      ptx::tc_fence_after();
#pragma unroll
      for (int ch = 0; ch < TT / CH; ++ch) {
        if (!ok) break;
        float acc[CH];
        {
          uint32_t d[CH];
          ptx::tmem_ld<CH>(taddr + ch * CH, d);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < CH; ++j) acc[j] = __uint_as_float(d[j]);
        }
        for (int a = 1; a < n_acc; ++a) {
          uint32_t d[CH];
          ptx::tmem_ld<CH>(taddr + a * TT + ch * CH, d);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < CH; ++j) acc[j] += __uint_as_float(d[j]);
        }
        if (ch == TT / CH - 1) {
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar_accempty);     // the accumulators may be overwritten
        }
        if constexpr (SPLITK == 2) {
          // cluster split-K: the partial waits in this CTA's own shared memory (the operand ring is idle: the
          // CTA's only unit is finished), [token column][128 weight rows]; the reduction follows below
          float* red = reinterpret_cast<float*>(smem) + row;
#pragma unroll
          for (int j = 0; j < CH; ++j) red[(ch * CH + j) * 128] = acc[j];
          continue;
        }
        if constexpr (SPLITK == 1) {
#pragma unroll
          for (int j = 0; j < CH; ++j) __stcg(part + (size_t)(ch * CH + j) * 128, acc[j]);
          continue;
        }
        const int m_left = p.M - (m_base + ch * CH);
        for (int t = 0; t < outs.n; ++t) {
          __nv_bfloat16* dst = outs.ptr[t] + (long long)(m_base + ch * CH) * p.ldc + n;
#pragma unroll
          for (int j = 0; j < CH; ++j) {
            if (j < m_left) *dst = __float2bfloat16_rn(acc[j]);
            dst += p.ldc;
          }
        }
      }
      if constexpr (SPLITK == 2) break;
      if constexpr (SPLITK == 1) {
        // The CTA that arrives last on the tile's counter adds all partials in split order (the same bits
        // whichever CTA that is) and writes the tile; the counter goes back to zero for the next call.
        __threadfence();
        ptx::bar_sync(1, 128);
        if (leader) {
          int verdict = 2;  // 2 = a wait gave up somewhere in this CTA: stop
          if (!ctl->abort) {
            const int old = atomicAdd(p.ws_counter + c.tile, 1);
            verdict = (old == p.split - 1) ? 1 : 0;
          }
          ctl->last = verdict;
        }
        ptx::bar_sync(1, 128);
        const int verdict = ctl->last;
        if (verdict == 2) break;
        if (verdict == 0) continue;
        __threadfence();
        mxs_reduce_tile<TT>(p.ws_partial + (size_t)c.tile * p.split * tile_floats + row, p.split, p.M, p.ldc, outs,
                            m_base, n);
        if (leader) atomicExch(p.ws_counter + c.tile, 0);
      }
    }
  }

  if constexpr (SPLITK == 2) {
    // ------------------------------------------------- cluster split-K reduction
    // Rank r adds the token columns [r, r+1) * TT / split of all ranks' partials in rank order (the order of
    // the workspace path: the same bits) and writes them.  A rank whose bounded wait gave up has parked
    // nothing: then no rank stores the tile.
    ptx::cluster_sync_all();             // every CTA's partial is in its shared memory
    if (warp >= 6 && blockIdx.x < p.num_units) {
      const UnitCoord c = decode_unit(blockIdx.x, p);
      uint32_t bad = 0;
      {
        const uint32_t abort_addr = ptx::smem_u32(&ctl->abort);
#pragma unroll
        for (int s = 0; s < 8; ++s)
          if (s < p.split) bad |= ptx::ld_cluster_u32(ptx::map_to_cta(abort_addr, s));
      }
      switch (p.split) {
        case 2: mxs_reduce_cols<TT, 2>(ring, warp & 3, lane, c, p, outs, bad); break;
        case 4: mxs_reduce_cols<TT, 4>(ring, warp & 3, lane, c, p, outs, bad); break;
        default: mxs_reduce_cols<TT, 8>(ring, warp & 3, lane, c, p, outs, bad); break;
      }
    }
    ptx::cluster_sync_all();             // no rank reads this CTA's shared memory any more
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (ctl->abort) __nanosleep(1000000);  // let copies that are still in flight land
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}

}  // namespace fp8mm
