// Decode path (one to a handful of tokens): block-scaled FP8 GEMV, a stream over the weights.
//
//   C[m,n] = sum_kb ( A[m, 128kb..] . B[n, 128kb..] ) * As[m,kb] * Bs[n/128,kb]      (bf16 out)
//
// With one to four tokens the call reads 1-25 MB of weights in the 1-4 us that a kernel launch
// costs anyway and does 2*M flop per weight byte against the ~560 flop/byte ridge of the part.
// What matters is that every SM pulls from the first cycle and that nothing stands between the
// load and the store.  The tcgen05 tiles (fp8mm_kernel.cuh) pay for tensor memory allocation,
// barrier set-up, tensor-map fetches and three role hand-offs per K block before the first byte
// of C leaves; here a warp loads weight rows straight into registers, widens them to f16
// (exact) and multiplies with FP32-accumulating FMAs: no tensor memory, no mbarriers, no tensor maps.
// (Register-level MMAs were measured as the alternative: on B200 mma.sync runs at about 220
// multiply-adds per clock and SM for f16 and slower still for e4m3, and its smallest tile has
// eight token columns, so for up to four tokens the FMAs are both fewer and faster.)
//
// Work decomposition: an item is 8 consecutive weight rows x 512 bytes of K (four 128-wide K
// blocks), one item per warp; lane l holds bytes [16 (l%8), +16) of K block l/8 of the chunk, so
// a row is one coalesced 512-byte load and the tokens' values for the lane's bytes live in
// registers.  The `kw` warps that cover the K chunks of a row group sit in the same CTA and add
// their sums in chunk order through shared memory; `groups` row groups share a CTA.  All
// additions run in a fixed order: the result does not depend on the SM count or timing.
//
// The math is the reference's (fp8_gemm_h20/kernels/kernel_v2.py:77-91,164-174): per K block a
// fresh FP32 dot product, one scale product As*Bs, FP32 accumulate, bf16 store.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "ptx_sm100.cuh"

namespace fp8mm {

constexpr int kGemvRows = 8;          // weight rows per item
constexpr int kGemvMaxWarps = 8;      // warps per CTA
constexpr int kGemvMaxTargets = 8;

struct GemvParams {
  const unsigned char* A;     // [M, K] e4m3
  const unsigned char* B;     // [N, K] e4m3
  const float* As;
  const float* Bs;
  __nv_bfloat16* out[kGemvMaxTargets];   // the caller's C and, for the fused all-gather, the peers' copies
  long long as_sm, as_sk, bs_sn, bs_sk, ldc;
  int n_out;
  int M, N, K;
  int kb_total;     // K / 128
  int n_kc;         // K chunks of four K blocks: ceil(kb_total / 4)
  int kw;           // warps per row group = min(n_kc, 8); a warp takes the chunks kw apart
  int groups;       // row groups per CTA pass; the CTA has kw * groups warps
  int n_rg;         // N / 8
  int ue8m0;        // As and Bs point to UE8M0 exponent bytes (value 2^(b-127)), strides in bytes
  int act_f32;      // ... but As holds floats after all (float32 powers of two from the quantiser)
};

// One scale: a float, or an exponent byte made into the float 2^(b-127) (b = 0 reads as 0).
__device__ __forceinline__ float gemv_scale(const float* base, long long at, int ue8m0) {
  if (ue8m0)
    return __uint_as_float(static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned char*>(base) + at)) << 23);
  return __ldg(base + at);
}

// Four e4m3 bytes -> two f16x2 registers (bytes 0,1 and bytes 2,3), exactly.
__device__ __forceinline__ void e4m3x4_to_f16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t"
      ".reg .b16 l, h;\n\t"
      "mov.b32 {l, h}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, l;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, h;\n\t"
      "}\n"
      : "=r"(lo), "=r"(hi)
      : "r"(w));
}
__device__ __forceinline__ void e4m3x16_to_f16(const uint4& raw, uint32_t (&h)[8]) {
  e4m3x4_to_f16x4(raw.x, h[0], h[1]);
  e4m3x4_to_f16x4(raw.y, h[2], h[3]);
  e4m3x4_to_f16x4(raw.z, h[4], h[5]);
  e4m3x4_to_f16x4(raw.w, h[6], h[7]);
}

// (e, o) += (w.lo * a.lo, w.hi * a.hi): two FP32 FMAs whose factors are the halves of two f16x2
// registers (mixed-precision fma.rn.f32.f16: f16 x f16 + f32, exact product, one rounding).
__device__ __forceinline__ void fma_f16x2_f32(float& e, float& o, uint32_t w, uint32_t a) {
  asm("{\n\t"
      ".reg .b16 wl, wh, al, ah;\n\t"
      "mov.b32 {wl, wh}, %2;\n\t"
      "mov.b32 {al, ah}, %3;\n\t"
      "fma.rn.f32.f16 %0, wl, al, %0;\n\t"
      "fma.rn.f32.f16 %1, wh, ah, %1;\n\t"
      "}\n"
      : "+f"(e), "+f"(o)
      : "r"(w), "r"(a));
}

// MT = tokens per warp (1, 2 or 4); blockIdx.y picks the token group.  One item per warp: the
// grid covers every (row group, K chunk) once, so that all loads of the call are in flight as
// early as the hardware can place the CTAs; registers are kept low for the same reason (warps
// per SM are what hides the load latency here).
template <int MT>
__global__ void __launch_bounds__(kGemvMaxWarps * 32, MT == 1 ? 3 : (MT == 2 ? 2 : 1))
fp8mm_gemv_kernel(const GemvParams p) {
  constexpr int R = kGemvRows;
  __shared__ float red[kGemvMaxWarps][MT][R];   // [warp][token][row]

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int grp = warp / p.kw;          // row group slot inside the CTA
  const int kcw = warp - grp * p.kw;    // first K chunk of this warp
  const int j = lane >> 3;              // K block inside the chunk
  const int sub = lane & 7;             // 16-byte piece of the K block
  const int m0 = blockIdx.y * MT;
  const int rg = blockIdx.x * p.groups + grp;
  const bool live = rg < p.n_rg;

  // Nothing above reads global memory: under programmatic dependent launch everything from here
  // on waits for the previous kernel in the stream, and the next one may start its prologue.
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();

  float tot[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) tot[m] = 0.f;

  for (int kc = kcw; kc < p.n_kc && live; kc += p.kw) {
    const int kb = kc * 4 + j;
    const bool ok = kb < p.kb_total;
    // every load of the item in flight before the first use
    uint4 w[R];
    uint4 araw[MT];
    float as_reg[MT];
    float bs = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) w[r] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      araw[m] = make_uint4(0u, 0u, 0u, 0u);
      as_reg[m] = 0.f;
    }
    if (ok) {
      const unsigned char* src = p.B + (size_t)(rg * R) * p.K + (size_t)kb * 128 + sub * 16;
#pragma unroll
      for (int r = 0; r < R; ++r) w[r] = __ldg(reinterpret_cast<const uint4*>(src + (size_t)r * p.K));
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const int tok = min(m0 + m, p.M - 1);
        araw[m] = __ldg(reinterpret_cast<const uint4*>(p.A + (size_t)tok * p.K + (size_t)kb * 128 + sub * 16));
        as_reg[m] = gemv_scale(p.As, (long long)tok * p.as_sm + (long long)kb * p.as_sk, p.ue8m0 && !p.act_f32);
      }
      bs = gemv_scale(p.Bs, (long long)((rg * R) >> 7) * p.bs_sn + (long long)kb * p.bs_sk, p.ue8m0);
    }
    uint32_t act[MT][8];
#pragma unroll
    for (int m = 0; m < MT; ++m) e4m3x16_to_f16(araw[m], act[m]);

    // v[r][m] = dot of this lane's 16 products; even and odd k in separate chains, added at the end
    float v[R][MT];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      uint32_t wh[8];
      e4m3x16_to_f16(w[r], wh);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        float e = 0.f, o = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) fma_f16x2_f32(e, o, wh[i], act[m][i]);
        v[r][m] = e + o;
      }
    }

    // Sum over the eight lanes of a K block.  Butterfly that halves the rows a lane keeps at
    // every step (4 + 2 + 1 exchanges per token instead of 3 x 8): afterwards lane l holds the
    // K-block dot product of row l % 8.
    {
      const bool up = (lane & 4) != 0;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const float send = up ? v[i][m] : v[i + 4][m];
          const float keep = up ? v[i + 4][m] : v[i][m];
          v[i][m] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
        }
    }
    {
      const bool up = (lane & 2) != 0;
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const float send = up ? v[i][m] : v[i + 2][m];
          const float keep = up ? v[i + 2][m] : v[i][m];
          v[i][m] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
        }
    }
    {
      const bool up = (lane & 1) != 0;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float send = up ? v[0][m] : v[1][m];
        const float keep = up ? v[1][m] : v[0][m];
        v[0][m] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
      }
    }
    // promote with the K block's scale product, then add the chunk's four K blocks
    // ((0 + 1) + (2 + 3)); K blocks past the end of K contribute exact zeros
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float t = v[0][m] * (as_reg[m] * bs);
      t += __shfl_xor_sync(0xffffffffu, t, 8);
      t += __shfl_xor_sync(0xffffffffu, t, 16);
      tot[m] += t;
    }
  }

  // add the K chunks of the row group in chunk order, then store
  if (p.kw > 1) {
    if (live && lane < R) {
#pragma unroll
      for (int m = 0; m < MT; ++m) red[warp][m][lane] = tot[m];
    }
    ptx::bar_sync(1 + grp, p.kw * 32);
    if (live && kcw == 0 && lane < R) {
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        float sum = red[warp][m][lane];
        for (int x = 1; x < p.kw; ++x) sum += red[warp + x][m][lane];
        tot[m] = sum;
      }
    }
  }
  if (live && kcw == 0 && lane < R) {
    const int n = rg * R + lane;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m0 + m < p.M) {
        const __nv_bfloat16 b = __float2bfloat16_rn(tot[m]);
        for (int d = 0; d < p.n_out; ++d) p.out[d][(long long)(m0 + m) * p.ldc + n] = b;
      }
    }
  }
}

}  // namespace fp8mm
