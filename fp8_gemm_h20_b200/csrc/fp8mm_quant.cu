// Activation quantiser: bf16 X[M,K] -> e4m3 A[M,K] + fp32 As[M,K/128], one scale per 1x128 group.
//
// This is the step right before the GEMM.  The reference leaves it to SGLang
// (sgl_patch/fp8mm_sglang_patch.py:53, sglang_per_token_group_quant_fp8 with row-major scales)
// and restates the recipe for its synthetic inputs in scripts/validate.py:26-28:
//   scale = max(amax(|x|) over the group, floor) / 448,  a = cast_e4m3(clamp(x / scale, +-448)).
// HBM-bound (3 bytes per element): 16-byte loads, 8-byte stores, one half-warp per group, the
// group maximum through shuffles, IEEE division and round-to-nearest-even conversion so the
// bytes equal what torch produces for the same recipe.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/fp8mm_b200.h"

namespace {

// POW2: the scale is rounded UP to a power of two and stored as its UE8M0 exponent byte (value
// 2^(b-127)), the form the block-scaled tensor-core kernels take (SGLang's quantiser with
// scale_ue8m0=True follows the same rule).
template <bool POW2>
__global__ void __launch_bounds__(256) quantize_act_kernel(const __nv_bfloat16* __restrict__ x,
                                                           uint8_t* __restrict__ a, void* __restrict__ as_,
                                                           int M, int K, long long ldx, long long as_sm,
                                                           long long as_sk, float floor_) {
  const int groups_per_row = K >> 7;
  const long long total = (long long)M * groups_per_row;
  const int sub = threadIdx.x & 15;                       // 16 threads x 8 elements = one group
  const int half = (threadIdx.x >> 4) & 1;                // two groups per warp
  const long long warp_first = (((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5) * 2;
  const long long step = ((long long)gridDim.x * blockDim.x) >> 4;
  // whole warps iterate together (the shuffles below name all 32 lanes); a half-warp whose
  // group lies past the end computes on zeros and stores nothing
  for (long long g0 = warp_first; g0 < total; g0 += step) {
    const long long g = g0 + half;
    const bool valid = g < total;
    const int m = valid ? (int)(g / groups_per_row) : 0;
    const int kb = valid ? (int)(g - (long long)m * groups_per_row) : 0;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (valid) raw = *reinterpret_cast<const uint4*>(x + (long long)m * ldx + kb * 128 + sub * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float v[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o, 16));
    float scale = __fdiv_rn(fmaxf(amax, floor_), 448.f);
    uint32_t ebyte = 0;
    if (POW2) {
      const uint32_t bits = __float_as_uint(scale);          // positive and normal: floor_ > 0
      ebyte = min(((bits >> 23) & 0xFFu) + ((bits & 0x7FFFFFu) != 0u ? 1u : 0u), 254u);
      scale = __uint_as_float(ebyte << 23);
    }
    uint2 packed;
    uint16_t* out16 = reinterpret_cast<uint16_t*>(&packed);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 q;
      q.x = fminf(fmaxf(__fdiv_rn(v[2 * i], scale), -448.f), 448.f);
      q.y = fminf(fmaxf(__fdiv_rn(v[2 * i + 1], scale), -448.f), 448.f);
      out16[i] = __nv_cvt_float2_to_fp8x2(q, __NV_SATFINITE, __NV_E4M3);
    }
    if (valid) {
      *reinterpret_cast<uint2*>(a + (long long)m * K + kb * 128 + sub * 8) = packed;
      if (sub == 0) {
        const long long at = (long long)m * as_sm + (long long)kb * as_sk;
        if (POW2) static_cast<uint8_t*>(as_)[at] = static_cast<uint8_t>(ebyte);
        else static_cast<float*>(as_)[at] = scale;
      }
    }
  }
}

}  // namespace

static int quantize_act(bool pow2, const void* x_bf16, void* a_e4m3, void* as, int32_t M, int32_t K, int64_t ldx,
                        int64_t as_stride_m, int64_t as_stride_k, float floor_, void* stream) {
  if (x_bf16 == nullptr || a_e4m3 == nullptr || as == nullptr) return FP8MM_E_NULL;
  if (!(floor_ > 0.f)) return FP8MM_E_CONFIG;
  if (M < 1 || K < 128 || (K % 128) != 0) return FP8MM_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(a_e4m3) & 7) || ldx < K ||
      (ldx % 8) != 0)
    return FP8MM_E_ALIGN;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
    return FP8MM_E_DRIVER;
  const long long groups = (long long)M * (K / 128);
  long long blocks = (groups * 16 + 255) / 256;
  const long long cap = (long long)sms * 8;               // 8 resident CTAs of 256 threads per SM
  if (blocks > cap) blocks = cap;
  if (pow2)
    quantize_act_kernel<true><<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x_bf16), static_cast<uint8_t*>(a_e4m3), as, M, K, ldx, as_stride_m,
        as_stride_k, floor_);
  else
    quantize_act_kernel<false><<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x_bf16), static_cast<uint8_t*>(a_e4m3), as, M, K, ldx, as_stride_m,
        as_stride_k, floor_);
  return cudaGetLastError() == cudaSuccess ? FP8MM_OK : FP8MM_E_LAUNCH;
}

extern "C" int fp8mm_b200_quantize_act(const void* x_bf16, void* a_e4m3, float* as, int32_t M, int32_t K,
                                       int64_t ldx, int64_t as_stride_m, int64_t as_stride_k, float floor_,
                                       void* stream) {
  return quantize_act(false, x_bf16, a_e4m3, as, M, K, ldx, as_stride_m, as_stride_k, floor_, stream);
}

extern "C" int fp8mm_b200_quantize_act_ue8m0(const void* x_bf16, void* a_e4m3, uint8_t* as_e, int32_t M, int32_t K,
                                             int64_t ldx, int64_t as_stride_m, int64_t as_stride_k, float floor_,
                                             void* stream) {
  return quantize_act(true, x_bf16, a_e4m3, as_e, M, K, ldx, as_stride_m, as_stride_k, floor_, stream);
}

// ------------------------------------------------------------------ UE8M0 scale expansion
// UE8M0 is the 8-bit exponent-only scale format of Blackwell block-scaled MMA and of DeepGEMM's
// sm_100 path: value = 2^(e - 127).  SGLang on Blackwell re-quantises block-FP8 weight scales to
// it and packs four consecutive K-block exponents into one int32, MN-major.  The GEMM of this
// library takes FP32 scales, so the packed form is expanded once per weight (exact: a power of two
// is an FP32 bit pattern).  e = 0 gives the subnormal 2^-127, e = 255 (NaN in the format) gives a
// quiet NaN.
__global__ void expand_ue8m0_kernel(const uint8_t* __restrict__ src, float* __restrict__ dst, int rows,
                                    int kblocks, long long row_stride, long long col_stride, int packed4) {
  const long long total = (long long)rows * kblocks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / kblocks), kb = (int)(i - (long long)r * kblocks);
    uint32_t e;
    if (packed4) {
      // strides count int32 words; byte kb%4 of the word (little endian) is K block kb
      const long long w = (long long)r * row_stride + (long long)(kb >> 2) * col_stride;
      e = src[w * 4 + (kb & 3)];
    } else {
      e = src[(long long)r * row_stride + (long long)kb * col_stride];
    }
    const uint32_t bits = e == 0u ? 0x00400000u : (e == 255u ? 0x7FC00000u : (e << 23));
    dst[i] = __uint_as_float(bits);
  }
}

extern "C" int fp8mm_b200_expand_ue8m0(const void* src, float* dst, int32_t rows, int32_t kblocks,
                                       int64_t row_stride, int64_t col_stride, int32_t packed4, void* stream) {
  if (src == nullptr || dst == nullptr) return FP8MM_E_NULL;
  if (rows < 1 || kblocks < 1) return FP8MM_E_SHAPE;
  if (packed4 != 0 && (reinterpret_cast<uintptr_t>(src) & 3)) return FP8MM_E_ALIGN;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
    return FP8MM_E_DRIVER;
  const long long total = (long long)rows * kblocks;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sms * 8;               // 8 resident CTAs of 256 threads per SM
  if (blocks > cap) blocks = cap;
  expand_ue8m0_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), dst, rows, kblocks, row_stride, col_stride, packed4);
  return cudaGetLastError() == cudaSuccess ? FP8MM_OK : FP8MM_E_LAUNCH;
}
