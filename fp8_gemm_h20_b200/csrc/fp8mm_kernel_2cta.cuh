// Two-CTA (cta_group::2) variant of the block-scaled FP8 GEMM for large token counts.
//
// A CTA pair computes a 256 (tokens) x 256 (weights) tile with tcgen05.mma.cta_group::2: each
// CTA loads only its own 128 token rows and its own HALF of the weight tile (32 KB per K block
// instead of 48 KB for the same MMA work per SM); the tensor cores read the other half of B
// from the partner's shared memory.  Every load is an ordinary single-destination
// cp.async.bulk.tensor issued by the CTA that owns the bytes.
//
// It is bit-equal to the one-CTA 128x256 kernel.  With per-K-block promotion the pace of both
// kernels is set by the loop around a TMEM accumulator buffer (MMAs issued -> promotion warps
// awake -> loads landed -> buffer released -> issuer sees it empty); the pair saves operand
// traffic but its release crosses from the partner SM to the leader's barrier, which lengthens
// that loop.  Available as impl "umma_2cta"; the tuner decides where it is used.
//
// Roles per CTA are those of fp8mm_umma_kernel (TMA producer, MMA issuer, scale loader, eight
// promotion/epilogue warps).  Differences:
//   * only the leader CTA (cluster rank 0) issues MMAs (two threads, alternate K blocks); its `full`
//     barrier collects the transaction bytes of both CTAs' loads (the partner's TMA signals the
//     leader's barrier);
//   * two tcgen05.commit per K block, each multicast to both CTAs: `tfull` (the promotion warps)
//     and `empty` (each CTA's producer gets its ring slot back);
//   * the leader's `tempty` barrier counts the promotion warps of both CTAs (the partner's
//     arrive through the cluster shared-memory window);
//   * TMEM is allocated and freed with the cta_group::2 forms by the same warp of both CTAs;
//   * cluster barriers bracket the kernel so that neither CTA touches the other's barriers
//     before they exist or exits while the other may still signal them.
#pragma once
#include "fp8mm_kernel.cuh"

namespace fp8mm {
namespace ptx {

__device__ __forceinline__ void tmem_alloc_2cta(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2cta() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// TMA load of this CTA's bytes; completion is counted on `bar`, which may be the leader's.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f8_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrive on the barrier at this offset in every CTA of `mask` once the MMAs have retired.
__device__ __forceinline__ void umma_commit_2cta(uint32_t bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(mask)
      : "memory");
}
__host__ __device__ constexpr uint32_t idesc_f8_m256(uint32_t n) {
  return (1u << 4) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}

}  // namespace ptx

struct Pair2Cta {
  static constexpr int UMMA_N = 256;
  static constexpr int NPW = 8;
  static constexpr int CPT = 128;
  static constexpr int CH = 32;
  static constexpr int NCH = CPT / CH;
  static constexpr int THREADS = kProducerThreads + NPW * 32;
  static constexpr uint32_t A_BYTES = 128u * 128u;        // this CTA's 128 token rows
  static constexpr uint32_t B_BYTES = 128u * 128u;        // this CTA's half of the 256 weight rows
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t STAGING_BYTES = NPW * 4096u;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Pair2Cta::THREADS, 1)
fp8mm_umma_2cta_kernel(const __grid_constant__ CUtensorMap tm_tok,
                       const __grid_constant__ CUtensorMap tm_wgt,
                       const __grid_constant__ OutTargets outs, const KParams p) {
  using T = Pair2Cta;
  constexpr int UMMA_N = T::UMMA_N, NPW = T::NPW, CPT = T::CPT, CH = T::CH, NCH = T::NCH;
  constexpr uint32_t STAGE_BYTES = T::STAGE_BYTES, A_BYTES = T::A_BYTES;
  constexpr uint32_t IDESC = ptx::idesc_f8_m256(UMMA_N);
  constexpr int TT = 128;                      // token rows of this CTA

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  unsigned char* smem = smem_raw + pad;
  const uint32_t ring = raw_addr + pad;

  const int kbn = p.kb_per_unit;
  const int stages = p.stages;
  const uint32_t staging = ring + stages * STAGE_BYTES;
  unsigned char* staging_ptr = smem + (size_t)stages * STAGE_BYTES;
  float* tab_a = reinterpret_cast<float*>(staging_ptr + T::STAGING_BYTES);   // [2][kbn][128]
  float* tab_b = tab_a + 2 * kbn * TT;                                        // [2][kbn][2]
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(tab_b + 2 * kbn * 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();       // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;

  const uint32_t bar_full = ptx::smem_u32(&ctl->full[0]);
  const uint32_t bar_empty = ptx::smem_u32(&ctl->empty[0]);
  const uint32_t bar_tfull = ptx::smem_u32(&ctl->tfull[0]);
  const uint32_t bar_tempty = ptx::smem_u32(&ctl->tempty[0]);
  const uint32_t bar_scfull = ptx::smem_u32(&ctl->scfull[0]);
  const uint32_t bar_scempty = ptx::smem_u32(&ctl->scempty[0]);
  // the leader's copies, as seen from this CTA
  const uint32_t lead_full = ptx::map_to_cta(bar_full, 0);
  const uint32_t lead_tempty = ptx::map_to_cta(bar_tempty, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_tfull + 8 * b, 1);
      ptx::mbar_init(bar_tempty + 8 * b, 2 * NPW);      // promotion warps of both CTAs
      ptx::mbar_init(bar_scfull + 8 * b, 64);
      ptx::mbar_init(bar_scempty + 8 * b, NPW);
    }
    ctl->abort = 0;
    ctl->last = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tm_tok);
    ptx::prefetch_tensormap(&tm_wgt);
    for (int d = 0; d < outs.n; ++d) ptx::prefetch_tensormap(&outs.map[d]);
  }
  if (warp == 1) {
    ptx::tmem_alloc_2cta(ptx::smem_u32(&ctl->tmem_base), T::TMEM_COLS);
    ptx::tmem_relinquish_2cta();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();          // both CTAs' barriers exist before anyone signals across
  ptx::tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();

  BoundedWait bw{&ctl->abort, p.status, p.timeout_ns};

  if (warp < 4) {
    ptx::setmaxnreg_dec<56>();
    if (warp == 0) {
      // ---------------------------------------------------------- TMA producer (both CTAs)
      if (lane == 0) {
        int stage = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int u = pair; u < p.num_units && ok; u += pairs) {
          const UnitCoord c = decode_unit(u, p);
          const int tok_y = c.ti * 256 + (int)rank * 128;
          const int wgt_y = c.wi * 256 + (int)rank * 128;
          for (int kb = 0; kb < kbn; ++kb) {
            if (!bw.wait(bar_empty + 8 * stage, ph ^ 1u, kWaitProducerEmpty)) { ok = false; break; }
            const uint32_t dst = ring + stage * STAGE_BYTES;
            // the leader announces the bytes of both CTAs; both CTAs' copies complete on its barrier
            if (rank == 0) ptx::mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * STAGE_BYTES);
            ptx::tma_load_2d_pair(dst, &tm_tok, lead_full + 8 * stage, kb * 128, tok_y);
            ptx::tma_load_2d_pair(dst + A_BYTES, &tm_wgt, lead_full + 8 * stage, kb * 128, wgt_y);
            if (++stage == stages) { stage = 0; ph ^= 1u; }
          }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer (leader only)
      if (lane == 0 && rank == 0) {
        int stage = 0;
        uint32_t ph = 0, it = 0;
        bool ok = true;
        for (int u = pair; u < p.num_units && ok; u += pairs) {
          for (int kb = 0; kb < kbn; ++kb, ++it) {
            const uint32_t buf = it & 1u, tph = (it >> 1) & 1u;
            if (!bw.wait(bar_full + 8 * stage, ph, kWaitMmaFull)) { ok = false; break; }
            if (!bw.wait(bar_tempty + 8 * buf, tph ^ 1u, kWaitMmaTmemEmpty)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint32_t a_addr = ring + stage * STAGE_BYTES;
            const uint64_t a_desc = ptx::smem_desc_k128(a_addr);
            const uint64_t b_desc = ptx::smem_desc_k128(a_addr + A_BYTES);
            const uint32_t d_tmem = tmem_base + buf * UMMA_N;
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k)
              ptx::umma_f8_2cta(d_tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, k);
            ptx::umma_commit_2cta(bar_tfull + 8 * buf, 0x3);   // both CTAs' promotion warps
            ptx::umma_commit_2cta(bar_empty + 8 * stage, 0x3);  // both CTAs' producers: the slot is free
            if (++stage == stages) { stage = 0; ph ^= 1u; }
          }
        }
      }
      __syncwarp();
    } else {
      // -------------------------------------------------------------------- scale loader
      const int tid = threadIdx.x - 64;
      uint32_t ui = 0;
      for (int u = pair; u < p.num_units; u += pairs, ++ui) {
        const UnitCoord c = decode_unit(u, p);
        const uint32_t t = ui & 1u, tph = (ui >> 1) & 1u;
        if (!bw.wait(bar_scempty + 8 * t, tph ^ 1u, kWaitLoaderEmpty)) break;
        // this CTA's 128 token rows are token tile 2 * ti + rank of the 128-row grid; the first unit's
        // table is staged by the promotion warps (idle until the first MMAs retire)
        UnitCoord c2 = c;
        c2.ti = c.ti * 2 + (int)rank;
        if (ui > 0) stage_scales<128, 256, false, 64, 4>(tid, c2, p, kbn, tab_a + t * kbn * TT, tab_b + t * kbn * 2);
        ptx::mbar_arrive(bar_scfull + 8 * t);
      }
    }
  } else {
    // ------------------------------------------------------- promotion + epilogue warps
    ptx::setmaxnreg_inc<224>();
    const int pw = warp - 4;
    const int q = warp & 3;
    const int half = pw >> 2;
    const int row = q * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + half * CPT;
    const bool leader = threadIdx.x == kProducerThreads;
    uint32_t ui = 0, it = 0;
    for (int u = pair; u < p.num_units; u += pairs, ++ui) {
      const UnitCoord c = decode_unit(u, p);
      const uint32_t t = ui & 1u, sph = (ui >> 1) & 1u;
      if (ui == 0) {
        UnitCoord c2 = c;
        c2.ti = c.ti * 2 + (int)rank;
        stage_scales<128, 256, false, NPW * 32, 8>(threadIdx.x - kProducerThreads, c2, p, kbn, tab_a, tab_b);
        ptx::bar_sync(1, NPW * 32);
      }
      bool ok = bw.wait(bar_scfull + 8 * t, sph, kWaitPromoScale);
      const float* ta = tab_a + t * kbn * TT;
      const float* tb = tab_b + t * kbn * 2;

      float acc[CPT];
#pragma unroll
      for (int j = 0; j < CPT; ++j) acc[j] = 0.f;

      for (int kb = 0; kb < kbn && ok; ++kb, ++it) {
        const uint32_t buf = it & 1u, tph = (it >> 1) & 1u;
        const float sc = ta[kb * TT + row] * tb[kb * 2 + half];
        if (!bw.wait(bar_tfull + 8 * buf, tph, kWaitPromoTmemFull)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t taddr = lane_base + buf * UMMA_N;
        // 128 columns per thread in two waits; packed FP32 FMAs (same bits as fmaf); the buffer goes
        // back to the leader as soon as this warp's loads have landed (fp8mm_kernel.cuh has the why)
#define FP8MM_PAIR_CHUNK(dd_, ch_)                                                                  \
  _Pragma("unroll") for (int i_ = 0; i_ < CH; i_ += 2)                                              \
      ptx::ffma2(acc[(ch_) * CH + i_], acc[(ch_) * CH + i_ + 1], dd_[i_], dd_[i_ + 1], sc, sc)
        uint32_t d[2][CH];
        static_assert(NCH == 4, "two pairs of 32-column loads");
        ptx::tmem_ld<CH>(taddr, d[0]);
        ptx::tmem_ld<CH>(taddr + CH, d[1]);
        ptx::tmem_wait_ld();
        FP8MM_PAIR_CHUNK(d[0], 0);
        ptx::tmem_ld<CH>(taddr + 2 * CH, d[0]);
        FP8MM_PAIR_CHUNK(d[1], 1);
        ptx::tmem_ld<CH>(taddr + 3 * CH, d[1]);
        ptx::tmem_wait_ld();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(lead_tempty + 8 * buf);   // the leader issues the MMAs
        FP8MM_PAIR_CHUNK(d[0], 2);
        FP8MM_PAIR_CHUNK(d[1], 3);
#undef FP8MM_PAIR_CHUNK
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar_scempty + 8 * t);
      if (!ok) break;

      const int m0w = c.ti * 256 + (int)rank * 128 + q * 32;
      const int n0 = c.wi * 256 + half * CPT;
      if (m0w < p.M && n0 < p.N) {
        unsigned char* stg = staging_ptr + pw * 4096;
        const uint32_t stg_addr = staging + pw * 4096;
#pragma unroll
        for (int sl = 0; sl < CPT / 64; ++sl) {
          if (lane == 0) ptx::bulk_wait_read_all();
          __syncwarp();
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
            *reinterpret_cast<uint4*>(stg + lane * 128 + ((ck ^ (lane & 7)) << 4)) = o;
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            for (int d = 0; d < outs.n; ++d) ptx::tma_store_2d(&outs.map[d], stg_addr, n0 + sl * 64, m0w);
            ptx::bulk_commit_group();
          }
        }
      }
    }
    if (lane == 0) ptx::bulk_wait_all();   // stores (also those to peer GPUs) are done
    __syncwarp();
  }

  // ------------------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();          // the partner no longer signals this CTA's barriers
  if (warp == 1) {
    if (ctl->abort) __nanosleep(1000000);
    ptx::tc_fence_after();
    ptx::tmem_dealloc_2cta(tmem_base, T::TMEM_COLS);
  }
}

}  // namespace fp8mm
