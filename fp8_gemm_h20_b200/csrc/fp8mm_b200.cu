// Host side of the C ABI declared in include/fp8mm_b200.h: legality checks, split
// legalisation, workspace layout, TMA tensor-map cache and the kernel launch.
// Replaces the reference's per-kernel Python wrappers (fp8_gemm_h20/kernels/kernel_v2.py:339-376
// and siblings).  No torch, no allocation, no synchronisation on the launch path.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "../../include/fp8mm_b200.h"
#include "fp8mm_kernel.cuh"
#include "fp8mm_kernel_2cta.cuh"
#include "fp8mm_gemv.cuh"
#include "fp8mm_kernel_mx.cuh"

namespace fp8mm {
namespace {

// Workspace layout, identical for every call so that no call's fp32 partials can land where
// another call expects its (zero) counters: [status 256 B][counters kMaxSplitTiles x 4 B][partials].
constexpr size_t kStatusBytes = 256;
constexpr int kMaxSplitTiles = 16384;
constexpr size_t kCounterBytes = (size_t)kMaxSplitTiles * sizeof(int);
constexpr size_t kMaxDynSmem = 232448;       // 227 KB opt-in dynamic shared memory per CTA
constexpr int kMaxDevices = 64;
constexpr int kClusterUnschedulable = -100;   // internal: the cluster launch has no room, use the workspace


struct Geometry {
  int umma_n;       // UMMA N = columns of the accumulator tile
  bool swap;
  bool cluster;     // split-K reduced through a thread-block cluster instead of the workspace
  bool pair;        // CTA pairs (cta_group::2): 256 tokens per tile, each CTA loads half of B
  int tt, wt;       // token / weight tile
  int t_tiles, w_tiles, tiles;
  int kb_total, split, kbn;
  int stages;
  int threads;
  size_t smem;
  int stg_slabs;
  int kg;              // K blocks per ring slot (1..8)
  bool gemv;           // CUDA-core decode path: no tiles, no split, no scratch
  bool mx;             // UE8M0 scales through the block-scaled MMA (split-K on the swap-AB tiles only)
  size_t counter_bytes, partial_bytes;
};

bool is_pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }
bool cluster_split_allowed();

int check_cfg(int M, int N, int K, const fp8mm_cfg* c) {
  if (c == nullptr) return FP8MM_E_NULL;
  if (M < 1 || N < 128 || K < 128 || (N % 128) != 0 || (K % 128) != 0) return FP8MM_E_SHAPE;
  if ((c->flags & ~(FP8MM_FLAG_WORKSPACE_SPLIT | FP8MM_FLAG_K_PAIRS | FP8MM_FLAG_K_GROUP_MASK |
                    FP8MM_FLAG_SCALES_UE8M0 | FP8MM_FLAG_ACT_SCALES_F32)) != 0)
    return FP8MM_E_CONFIG;
  if ((c->flags & FP8MM_FLAG_ACT_SCALES_F32) &&
      !(c->impl == FP8MM_IMPL_UMMA_MX || (c->impl == FP8MM_IMPL_GEMV && (c->flags & FP8MM_FLAG_SCALES_UE8M0))))
    return FP8MM_E_CONFIG;
  // exponent-byte scales: the block-scaled kernels (always) and the decode kernel (on request)
  if ((c->flags & FP8MM_FLAG_SCALES_UE8M0) && c->impl != FP8MM_IMPL_GEMV && c->impl != FP8MM_IMPL_UMMA_MX)
    return FP8MM_E_CONFIG;
  if (c->split < 1 || c->group_m < 1 || c->stages < 0 || c->max_ctas < 0) return FP8MM_E_CONFIG;
  if (c->impl == FP8MM_IMPL_UMMA) {
    if (c->block_t != 128) return FP8MM_E_CONFIG;
    if (c->block_w != 128 && c->block_w != 256) return FP8MM_E_CONFIG;
  } else if (c->impl == FP8MM_IMPL_UMMA_SWAP) {
    if (c->block_w != 128) return FP8MM_E_CONFIG;
    if (!is_pow2(c->block_t) || c->block_t < 16 || c->block_t > 256) return FP8MM_E_CONFIG;
  } else if (c->impl == FP8MM_IMPL_UMMA_2CTA) {
    if (c->block_t != 256 || c->block_w != 256) return FP8MM_E_CONFIG;
  } else if (c->impl == FP8MM_IMPL_UMMA_MX) {
    const bool small = c->block_w == 128 && (c->block_t == 16 || c->block_t == 32 || c->block_t == 64 || c->block_t == 128);
    if (!((c->block_t == 128 && c->block_w == 256) || (c->block_t == 256 && c->block_w == 224) || small)) return FP8MM_E_CONFIG;
  } else if (c->impl == FP8MM_IMPL_GEMV) {
    if (c->block_w != kGemvRows) return FP8MM_E_CONFIG;
    if (c->block_t != 1 && c->block_t != 2 && c->block_t != 4) return FP8MM_E_CONFIG;
    if ((M + c->block_t - 1) / c->block_t > 65535) return FP8MM_E_CONFIG;
  } else {
    return FP8MM_E_CONFIG;
  }
  return FP8MM_OK;
}

// Tile counts, legalised split, ring depth and shared-memory size for one call.
int make_geometry(int M, int N, int K, const fp8mm_cfg* c, Geometry* g) {
  const int rc = check_cfg(M, N, K, c);
  if (rc != FP8MM_OK) return rc;
  memset(g, 0, sizeof(*g));
  g->gemv = c->impl == FP8MM_IMPL_GEMV;
  if (g->gemv) {             // one pass over the weights: nothing to legalise, no scratch
    g->split = 1;
    g->kb_total = g->kbn = K / 128;
    return FP8MM_OK;
  }
  if (c->impl == FP8MM_IMPL_UMMA_MX) {
    g->mx = true;
    if (c->block_w == 128) {
      // swap-AB: 128 weight rows x block_t tokens, plain stores (no output tensor map)
      g->swap = true;
      g->tt = c->block_t;
      g->wt = 128;
      g->umma_n = g->tt;
      g->t_tiles = (M + g->tt - 1) / g->tt;
      g->w_tiles = N / 128;
      g->tiles = g->t_tiles * g->w_tiles;
      g->kb_total = K / 128;
      g->kg = g->tt <= 64 ? 4 : 2;           // K blocks per ring slot = issuing threads (MxsTraits<TT>::NI)
      // FP8MM_FLAG_K_PAIRS on unsplit tiles: the half-size form (half the issuing threads, ring slot and tensor
      // memory), of which two CTAs share an SM
      const bool half_form = (c->flags & FP8MM_FLAG_K_PAIRS) && !(c->split > 1) && g->tt <= 64;
      if (half_form) g->kg = 2;
      // split-K: a split that does not divide the K-block count runs unsplit, like the table kernels'
      g->split = (c->split > 1 && g->kb_total % c->split == 0 && g->tiles <= kMaxSplitTiles) ? c->split : 1;
      g->kbn = g->kb_total / g->split;
      g->cluster = (g->split == 2 || g->split == 4 || g->split == 8) && cluster_split_allowed() &&
                   !(c->flags & FP8MM_FLAG_WORKSPACE_SPLIT);
      g->stg_slabs = 1;
      g->threads = 6 * 32 + 4 * 32;
      const size_t stage_bytes = (size_t)g->kg * (128 * 128 + (size_t)g->tt * 128);
      const size_t fixed = 1024 + 2 * 1024 + sizeof(MxCtl);
      int stages = c->stages > 0 ? c->stages : 4;
      const int fit = (int)((kMaxDynSmem - fixed) / stage_bytes);
      if (stages > fit) stages = fit;
      if (stages > kMaxStages) stages = kMaxStages;
      if (stages < 2) return FP8MM_E_CONFIG;
      g->stages = stages;
      // the cluster reduction parks the fp32 partial tile in the (then idle) operand ring
      if (g->cluster && (size_t)stages * stage_bytes < (size_t)g->tt * 128 * sizeof(float)) g->cluster = false;
      const bool ws_split = g->split > 1 && !g->cluster;
      g->counter_bytes = ws_split ? kCounterBytes : 0;
      g->partial_bytes = ws_split ? (size_t)g->tiles * g->split * g->tt * 128 * sizeof(float) : 0;
      size_t smem = fixed + (size_t)stages * stage_bytes;
      size_t tmem_cols = g->tt <= 16 ? 128 : (g->tt <= 32 ? 256 : 512);   // MxsTraits<TT, NI>::TMEM_COLS
      if (half_form) tmem_cols = g->tt <= 16 ? 64 : (g->tt <= 32 ? 128 : 256);
      const size_t floor_smem = tmem_cols * 456 - 1024;     // shared-memory share >= TMEM share (see below)
      g->smem = smem < floor_smem ? floor_smem : smem;
      return FP8MM_OK;
    }
    g->tt = c->block_t;
    g->wt = c->block_w;
    g->umma_n = g->wt;
    g->t_tiles = (M + g->tt - 1) / g->tt;
    g->w_tiles = (N + g->wt - 1) / g->wt;
    g->tiles = g->t_tiles * g->w_tiles;
    g->kb_total = g->kbn = K / 128;
    g->split = 1;
    g->kg = 1;
    g->stg_slabs = 2;
    g->threads = MxTraits::THREADS;
    const bool wide = g->tt == 256;
    const size_t stage_bytes = wide ? Mx256Traits::STAGE_BYTES : MxTraits::STAGE_BYTES;
    const size_t fixed = 1024 + sizeof(MxCtl) +
                         (wide ? Mx256Traits::STAGING_BYTES + 2 * Mx256Traits::SF_SLOT_BYTES
                               : MxTraits::STAGING_BYTES + 2 * MxTraits::SF_SLOT_BYTES);
    int stages = c->stages > 0 ? c->stages : 4;
    const int fit = (int)((kMaxDynSmem - fixed) / stage_bytes);
    if (stages > fit) stages = fit;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) return FP8MM_E_CONFIG;
    g->stages = stages;
    // the kernel takes all 512 TMEM columns, so it asks for all of the shared memory too: no other CTA
    // (of any stream) can then sit on the same SM waiting for tensor memory (the rule the tile kernels
    // follow: shared-memory share >= TMEM share)
    g->smem = kMaxDynSmem;
    return FP8MM_OK;
  }
  g->swap = c->impl == FP8MM_IMPL_UMMA_SWAP;
  g->pair = c->impl == FP8MM_IMPL_UMMA_2CTA;
  g->umma_n = g->swap ? c->block_t : c->block_w;
  g->tt = c->block_t;
  g->wt = c->block_w;
  g->t_tiles = (M + g->tt - 1) / g->tt;
  g->w_tiles = (N + g->wt - 1) / g->wt;
  g->tiles = g->t_tiles * g->w_tiles;
  g->kb_total = K / 128;
  // A split that does not divide the K-block count runs unsplit (kernel_v2.py:355-356).
  // So does a split over more tiles than the counter region holds (it could not pay off).
  g->split = (c->split > 1 && g->kb_total % c->split == 0 && g->tiles <= kMaxSplitTiles && !g->pair)
                 ? c->split : 1;
  g->kbn = g->kb_total / g->split;
  g->cluster = (g->split == 2 || g->split == 4 || g->split == 8) && cluster_split_allowed() &&
               !(c->flags & FP8MM_FLAG_WORKSPACE_SPLIT);
  const int npw = g->umma_n >= 128 ? 8 : 4;
  g->threads = kProducerThreads + npw * 32;
  // several K blocks per ring slot: narrow swap-AB tiles only, and only if the count divides every
  // split's K blocks (and two slots of that size fit into shared memory); otherwise one per slot
  int kg_req = (c->flags & FP8MM_FLAG_K_GROUP_MASK) >> 8;
  if (kg_req == 0 && (c->flags & FP8MM_FLAG_K_PAIRS)) kg_req = 2;
  g->kg = (kg_req >= 2 && kg_req <= 8 && g->swap && g->umma_n <= 64 && g->kbn % kg_req == 0) ? kg_req : 1;
  const size_t block_bytes = g->pair ? 2 * 128 * 128 : (128 * 128 + (size_t)g->umma_n * 128);
  const size_t tab_rows = g->pair ? 128 : g->tt;    // token rows per CTA in the scale table
  const size_t tab_bytes = 2 * (size_t)g->kbn * tab_rows * sizeof(float) + 2 * (size_t)g->kbn * 2 * sizeof(float);
  size_t staging = g->swap ? 0 : (size_t)npw * 4096;   // bf16 output staging for TMA stores
  size_t fixed = 1024 + staging + tab_bytes + sizeof(SharedCtl);
  if (fixed + 2 * g->kg * block_bytes > kMaxDynSmem) g->kg = 1;     // two slots of that size do not fit
  const size_t stage_bytes = g->kg * block_bytes;
  if (fixed + 2 * stage_bytes > kMaxDynSmem) return FP8MM_E_CONFIG;
  int stages = c->stages > 0 ? c->stages : (g->pair ? 5 : 4);
  if (stages > kMaxStages) stages = kMaxStages;
  // 256-wide token-major tiles: a second staging slab per epilogue warp (both column halves
  // staged and stored back to back) when it costs no ring stage
  g->stg_slabs = 1;
  if (!g->swap && !g->pair && g->umma_n == 256) {
    const int fit1 = (int)((kMaxDynSmem - fixed) / stage_bytes);
    const int want = stages < fit1 ? stages : fit1;
    if (fixed + staging + (size_t)want * stage_bytes <= kMaxDynSmem) {
      g->stg_slabs = 2;
      fixed += staging;
      staging *= 2;
    }
  }
  const int fit = (int)((kMaxDynSmem - fixed) / stage_bytes);
  if (stages > fit) stages = fit;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return FP8MM_E_CONFIG;
  g->stages = stages;
  // the cluster reduction parks the fp32 partial tile in the (then idle) operand ring
  // (token-major tiles park it row-major with rows padded by four floats)
  if (g->cluster && (size_t)stages * stage_bytes < (size_t)(g->umma_n + (g->swap ? 0 : 4)) * 128 * sizeof(float))
    g->cluster = false;
  size_t smem = fixed + stages * stage_bytes;
  // Shared memory share >= TMEM share, so that CTAs that fit on an SM together (this
  // kernel's or another stream's) can never ask for more than the 512 TMEM columns.
  const int nbuf = g->umma_n == 256 ? 2 : (g->umma_n >= 64 ? 4 : 8);   // KernelTraits::NBUF
  const size_t tmem_cols = nbuf * g->umma_n < 32 ? 32 : (size_t)nbuf * g->umma_n;
  const size_t floor_smem = tmem_cols * 456 - 1024;  // (smem + 1 KB reserved) / 228 KB >= cols / 512
  if (smem < floor_smem) smem = floor_smem;
  g->smem = smem;
  const bool ws_split = g->split > 1 && !g->cluster;
  g->counter_bytes = ws_split ? kCounterBytes : 0;
  g->partial_bytes = ws_split ? (size_t)g->tiles * g->split * g->umma_n * 128 * sizeof(float) : 0;
  return FP8MM_OK;
}

// ------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  int rows, k, box_rows;     // box_rows carries the K blocks per box in its upper bits
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && k == o.k && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= (size_t)k.rows * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= (size_t)k.k * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= (size_t)k.box_rows * 0x165667B19E3779F9ull + (h << 6) + (h >> 2);
    return h;
  }
};

std::mutex g_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// Row-major [rows, k] bytes, box = box_rows x 128 bytes, 128-byte swizzle, zero fill
// outside the tensor.  The encoding depends only on (pointer, shape, box): cached.
// kg = 2: the same bytes seen as a 3-D tensor (128 bytes, rows, K blocks) with a box of two K
// blocks, so that one copy delivers two consecutive operand tiles.
// Test hook (host side): FP8MM_TEST_SHORT_WEIGHT_BOX=1 encodes the WEIGHT operand's map with half the
// box rows, so that every weight copy delivers fewer bytes than the producer announced and the ring's
// `full` barrier never completes.  With a short FP8MM_TIMEOUT_MS the bounded waits then run out, the
// kernel records why and returns: the way the give-up path is exercised without a fault, a trap or an
// endless wait.  Read at every encode, so a test can switch it off again (maps are cached per pointer).
bool test_short_weight_box() {
  const char* e = getenv("FP8MM_TEST_SHORT_WEIGHT_BOX");
  return e != nullptr && e[0] == '1';
}

int get_tensor_map(const void* ptr, int rows, int k, int box_rows, CUtensorMap* out, int kg = 1,
                   bool weight = false) {
  const bool shorten = weight && test_short_weight_box();
  if (shorten) box_rows /= 2;
  const MapKey key{ptr, rows, k, box_rows | (kg << 16) | (shorten ? 1 << 30 : 0)};
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
      *out = it->second;
      return FP8MM_OK;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return FP8MM_E_DRIVER;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)k};
  cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUtensorMap m;
  CUresult r;
  if (kg == 1) {
    r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides,
           box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t dims3[3] = {128u, (cuuint64_t)rows, (cuuint64_t)(k / 128)};
    cuuint64_t strides3[2] = {(cuuint64_t)k, 128u};          // bytes: next row, next K block
    cuuint32_t box3[3] = {128u, (cuuint32_t)box_rows, (cuuint32_t)kg};
    cuuint32_t estr3[3] = {1u, 1u, 1u};
    r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims3, strides3,
           box3, estr3, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) return FP8MM_E_DRIVER;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_maps.size() > 8192) g_maps.clear();
    g_maps.emplace(key, m);
  }
  *out = m;
  return FP8MM_OK;
}

// bf16 C [M, N] with row stride ldc, box = 32 rows x 64 columns (128 bytes), 128-byte swizzle.
// Cached by (pointer, M, N, ldc) like the operand maps: a caching allocator hands the same output
// addresses out again and again, and an encode costs about as much as the rest of the host path.
struct OutKey {
  const void* ptr;
  int m, n;
  long long ldc;
  int narrow;     // 0: 64-column boxes, 128-byte swizzle; 1: 32-column boxes, 64-byte swizzle
  bool operator==(const OutKey& o) const {
    return ptr == o.ptr && m == o.m && n == o.n && ldc == o.ldc && narrow == o.narrow;
  }
};
struct OutKeyHash {
  size_t operator()(const OutKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= (size_t)k.m * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= (size_t)k.n * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= (size_t)k.ldc * 0x165667B19E3779F9ull + (h << 6) + (h >> 2);
    h ^= (size_t)k.narrow * 0x27D4EB2F165667C5ull;
    return h;
  }
};
std::unordered_map<OutKey, CUtensorMap, OutKeyHash> g_out_maps;

int make_output_map(void* c, int m, int n, long long ldc, CUtensorMap* out, bool narrow = false) {
  const OutKey key{c, m, n, ldc, narrow ? 1 : 0};
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_out_maps.find(key);
    if (it != g_out_maps.end()) {
      *out = it->second;
      return FP8MM_OK;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return FP8MM_E_DRIVER;
  cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)m};
  cuuint64_t strides[1] = {(cuuint64_t)ldc * 2};
  cuuint32_t box[2] = {narrow ? 32u : 64u, 32u};
  cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, narrow ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return FP8MM_E_DRIVER;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_out_maps.size() > 8192) g_out_maps.clear();
    g_out_maps.emplace(key, *out);
  }
  return FP8MM_OK;
}

// ----------------------------------------------------------------- launch
struct DeviceInfo {
  int sms = 0;
  bool attr_set[57] = {};     // 0..35 tile kernels, 39 CTA-pair kernel, 40/41 block-scaled (UE8M0) kernels
  // cluster split-K kernels: can a cluster of 2 / 4 / 8 such CTAs be placed at all?  0 = not asked
  // yet, 1 = yes, 2 = no (an SM-limited context, MPS or a green context can say no)
  unsigned char cluster_ok[54][4] = {};
};
DeviceInfo g_dev[kMaxDevices];

unsigned long long timeout_ns() {
  static unsigned long long v = []() {
    const char* e = getenv("FP8MM_TIMEOUT_MS");
    unsigned long long ms = e ? strtoull(e, nullptr, 10) : 2000ull;
    if (ms < 1) ms = 1;
    return ms * 1000000ull;
  }();
  return v;
}

// Programmatic dependent launch lets a kernel's prologue overlap the previous kernel's tail;
// FP8MM_PDL=0 turns it off.
bool use_pdl() {
  static const bool v = []() {
    const char* e = getenv("FP8MM_PDL");
    return !(e != nullptr && e[0] == '0');
  }();
  return v;
}

template <int UMMA_N, bool SWAP, int SPLITK, int KG = 1>
int launch_one(int slot, int dev, const Geometry& g, const CUtensorMap& tm_tok, const CUtensorMap& tm_wgt,
               const OutTargets& outs, const KParams& p, int grid, cudaStream_t stream) {
  auto kern = fp8mm_umma_kernel<UMMA_N, SWAP, SPLITK, KG>;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_dev[dev].attr_set[slot]) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxDynSmem) !=
          cudaSuccess)
        return FP8MM_E_LAUNCH;
      g_dev[dev].attr_set[slot] = true;
    }
  }
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(grid);
  lc.blockDim = dim3(g.threads);
  lc.dynamicSmemBytes = g.smem;
  lc.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (use_pdl()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (SPLITK == 2) {                       // the split CTAs of a tile form one cluster
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = g.split;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  lc.attrs = attr;
  lc.numAttrs = na;
  if (SPLITK == 2) {
    const int si = g.split == 2 ? 0 : (g.split == 4 ? 1 : 2);
    unsigned char known;
    {
      std::lock_guard<std::mutex> lk(g_mu);
      known = g_dev[dev].cluster_ok[slot][si];
    }
    if (known == 0) {
      int n = 0;
      const cudaError_t q = cudaOccupancyMaxActiveClusters(&n, kern, &lc);
      if (q != cudaSuccess) (void)cudaGetLastError();
      known = (q == cudaSuccess && n > 0) ? 1 : 2;
      std::lock_guard<std::mutex> lk(g_mu);
      g_dev[dev].cluster_ok[slot][si] = known;
    }
    if (known == 2) return kClusterUnschedulable;
  }
  const cudaError_t e = cudaLaunchKernelEx(&lc, kern, tm_tok, tm_wgt, outs, p);
  if (e != cudaSuccess) (void)cudaGetLastError();
  return e == cudaSuccess ? FP8MM_OK : FP8MM_E_LAUNCH;
}

// The kernels that exist in one form only: the CTA-pair kernel (slot 39) and the block-scaled one (40).
typedef void (*PlainKernel)(const CUtensorMap, const CUtensorMap, const OutTargets, const KParams);
int launch_plain(PlainKernel kern, int slot, int dev, const Geometry& g, const CUtensorMap& tm_tok,
                 const CUtensorMap& tm_wgt, const OutTargets& outs, const KParams& p, int grid, cudaStream_t stream,
                 int cluster = 0) {
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_dev[dev].attr_set[slot]) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxDynSmem) !=
          cudaSuccess)
        return FP8MM_E_LAUNCH;
      g_dev[dev].attr_set[slot] = true;
    }
  }
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(grid);
  lc.blockDim = dim3(g.threads);
  lc.dynamicSmemBytes = g.smem;
  lc.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (use_pdl()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (cluster > 1) {                       // the split CTAs of a tile form one cluster
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = cluster;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  lc.attrs = attr;
  lc.numAttrs = na;
  if (cluster > 1) {
    const int si = cluster == 2 ? 0 : (cluster == 4 ? 1 : 2);
    unsigned char known;
    {
      std::lock_guard<std::mutex> lk(g_mu);
      known = g_dev[dev].cluster_ok[slot][si];
    }
    if (known == 0) {
      int n = 0;
      const cudaError_t q = cudaOccupancyMaxActiveClusters(&n, kern, &lc);
      if (q != cudaSuccess) (void)cudaGetLastError();
      known = (q == cudaSuccess && n > 0) ? 1 : 2;
      std::lock_guard<std::mutex> lk(g_mu);
      g_dev[dev].cluster_ok[slot][si] = known;
    }
    if (known == 2) return kClusterUnschedulable;
  }
  const cudaError_t e = cudaLaunchKernelEx(&lc, kern, tm_tok, tm_wgt, outs, p);
  if (e != cudaSuccess) (void)cudaGetLastError();
  return e == cudaSuccess ? FP8MM_OK : FP8MM_E_LAUNCH;
}

// Split-K through a cluster (distributed shared memory) when the split is 2, 4 or 8, else
// through the workspace.  FP8MM_SPLIT_MODE=workspace forces the workspace path.
bool cluster_split_allowed() {
  static const bool v = []() {
    const char* e = getenv("FP8MM_SPLIT_MODE");
    return !(e != nullptr && e[0] == 'w');
  }();
  return v;
}

template <int UMMA_N, bool SWAP>
int launch(int slot, int dev, const Geometry& g, const CUtensorMap& tm_tok, const CUtensorMap& tm_wgt,
           const OutTargets& outs, const KParams& p, int grid, cudaStream_t stream) {
  if constexpr (SWAP && UMMA_N <= 64) {
    if (g.kg >= 2) {          // slots 21..29: the several-K-blocks-per-slot variants of the narrow tiles
      const int s2 = 21 + 3 * slot;
      if (g.split > 1) {
        if (g.cluster) {
          const int rc = launch_one<UMMA_N, SWAP, 2, 2>(s2 + 2, dev, g, tm_tok, tm_wgt, outs, p, p.num_units, stream);
          if (rc != kClusterUnschedulable) return rc;
          if (p.ws_partial == nullptr) return FP8MM_E_WORKSPACE;
        }
        return launch_one<UMMA_N, SWAP, 1, 2>(s2 + 1, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
      }
      return launch_one<UMMA_N, SWAP, 0, 2>(s2, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
    }
  }
  if (g.split > 1) {
    if (g.cluster) {
      // No room for a cluster of `split` CTAs in this context: the workspace reduction gives the same
      // bits, provided the caller's workspace is large enough for it (fp8mm_b200_workspace_bytes with
      // FP8MM_FLAG_WORKSPACE_SPLIT set says how large).
      const int rc = launch_one<UMMA_N, SWAP, 2>(3 * slot + 2, dev, g, tm_tok, tm_wgt, outs, p, p.num_units, stream);
      if (rc != kClusterUnschedulable) return rc;
      if (p.ws_partial == nullptr) return FP8MM_E_WORKSPACE;
    }
    return launch_one<UMMA_N, SWAP, 1>(3 * slot + 1, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
  }
  return launch_one<UMMA_N, SWAP, 0>(3 * slot, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
}

// Decode path: grid and CTA shape from the problem alone (see fp8mm_gemv.cuh).
template <int MT>
int launch_gemv_mt(const GemvParams& p, dim3 grid, int warps, cudaStream_t stream) {
  cudaLaunchConfig_t lc = {};
  lc.gridDim = grid;
  lc.blockDim = dim3(warps * 32);
  lc.dynamicSmemBytes = 0;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  int na = 0;
  if (use_pdl()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  lc.attrs = attr;
  lc.numAttrs = na;
  const cudaError_t e = cudaLaunchKernelEx(&lc, fp8mm_gemv_kernel<MT>, p);
  if (e != cudaSuccess) (void)cudaGetLastError();
  return e == cudaSuccess ? FP8MM_OK : FP8MM_E_LAUNCH;
}

int launch_gemv(int dev, const fp8mm_args* a, const fp8mm_cfg* cfg, void* const* extra_c, int n_extra,
                cudaStream_t stream) {
  const int sms = g_dev[dev].sms;
  const int mt = cfg->block_t;
  (void)cfg->max_ctas;     // one item per warp: the grid is the problem
  GemvParams p;
  memset(&p, 0, sizeof(p));
  p.A = static_cast<const unsigned char*>(a->A);
  p.B = static_cast<const unsigned char*>(a->B);
  p.As = a->As;
  p.Bs = a->Bs;
  p.ue8m0 = (cfg->flags & FP8MM_FLAG_SCALES_UE8M0) ? 1 : 0;
  p.act_f32 = (cfg->flags & FP8MM_FLAG_ACT_SCALES_F32) ? 1 : 0;
  p.n_out = 1 + n_extra;
  for (int d = 0; d < p.n_out; ++d) p.out[d] = static_cast<__nv_bfloat16*>(d == 0 ? a->C : extra_c[d - 1]);
  p.as_sm = a->as_stride_m;
  p.as_sk = a->as_stride_k;
  p.bs_sn = a->bs_stride_n;
  p.bs_sk = a->bs_stride_k;
  p.ldc = a->ldc;
  p.M = a->M;
  p.N = a->N;
  p.K = a->K;
  p.kb_total = a->K / 128;
  p.n_kc = (p.kb_total + 3) / 4;
  p.kw = p.n_kc < kGemvMaxWarps ? p.n_kc : kGemvMaxWarps;
  p.n_rg = a->N / kGemvRows;
  // row groups per CTA: as many as fit in eight warps, fewer while that leaves SMs without a CTA
  int groups = kGemvMaxWarps / p.kw;
  while (groups > 1 && (p.n_rg + groups - 1) / groups < 2 * sms) groups >>= 1;
  p.groups = groups;
  const int warps = p.kw * groups;
  const int grid_x = (p.n_rg + groups - 1) / groups;
  const dim3 grid(grid_x, (a->M + mt - 1) / mt);
  switch (mt) {
    case 1: return launch_gemv_mt<1>(p, grid, warps, stream);
    case 2: return launch_gemv_mt<2>(p, grid, warps, stream);
    case 4: return launch_gemv_mt<4>(p, grid, warps, stream);
  }
  return FP8MM_E_CONFIG;
}

}  // namespace
}  // namespace fp8mm

// ----------------------------------------------------- allocation-free entry point
// Scratch for callers that cannot allocate: status word, split-K tile counters and fp32 partial
// tiles in a buffer that is part of the library image.  Zero at load; the counters are re-zeroed by
// every call, the status word stays until it is fetched.  In host code `g_static_scratch` is only a handle for cudaGetSymbolAddress — the
// device address it yields is what the kernels receive.
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static void* g_static_scratch_addr[fp8mm::kMaxDevices] = {};  // per device, filled on first use


using namespace fp8mm;

extern "C" {

int fp8mm_b200_version(void) { return 1000; }

const char* fp8mm_b200_strerror(int code) {
  switch (code) {
    case FP8MM_OK: return "ok";
    case FP8MM_E_NULL: return "a required pointer is NULL";
    case FP8MM_E_SHAPE: return "M must be >= 1 and N, K multiples of 128";
    case FP8MM_E_CONFIG: return "illegal tile/split/stage configuration";
    case FP8MM_E_WORKSPACE: return "workspace missing or too small";
    case FP8MM_E_ALIGN: return "A, B and C must be 16-byte aligned and ldc a multiple of 8";
    case FP8MM_E_DRIVER: return "CUDA driver call failed (tensor map encode)";
    case FP8MM_E_LAUNCH: return "kernel launch failed";
    case FP8MM_E_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case FP8MM_E_TOO_LARGE:
      return "problem needs more scratch than the 8 MiB built into the allocation-free entry point";
    default: return "unknown error";
  }
}

int fp8mm_b200_validate(int32_t M, int32_t N, int32_t K, const fp8mm_cfg* cfg) {
  Geometry g;
  return make_geometry(M, N, K, cfg, &g);
}

size_t fp8mm_b200_workspace_bytes(int32_t M, int32_t N, int32_t K, const fp8mm_cfg* cfg) {
  Geometry g;
  if (make_geometry(M, N, K, cfg, &g) != FP8MM_OK) return 0;
  return kStatusBytes + g.counter_bytes + g.partial_bytes;
}

int fp8mm_b200_workspace_init(void* workspace, size_t ws_bytes, void* stream) {
  if (workspace == nullptr) return FP8MM_E_NULL;
  return cudaMemsetAsync(workspace, 0, ws_bytes, static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? FP8MM_OK
             : FP8MM_E_DRIVER;
}

static int static_scratch_address(void** out);

int fp8mm_b200_last_status(const void* workspace, int32_t* detail) {
  if (workspace == nullptr) {
    // callers of fp8mm_b200_gemm_static_scratch have no workspace pointer: NULL names the built-in
    // scratch of the current device
    void* scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != FP8MM_OK) return rc;
    workspace = scratch;
  }
  int32_t v = 0;
  if (cudaMemcpy(&v, workspace, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return FP8MM_E_DRIVER;
  if (detail != nullptr) *detail = v;
  return v == 0 ? FP8MM_OK : FP8MM_E_DEVICE_TIMEOUT;
}

static int gemm_impl(const fp8mm_args* a, const fp8mm_cfg* cfg, void* workspace, size_t ws_bytes,
                     void* stream_, void* const* extra_c, int n_extra) {
  if (n_extra < 0 || n_extra > kMaxOutTargets - 1 || (n_extra > 0 && extra_c == nullptr)) return FP8MM_E_CONFIG;
  if (a == nullptr || cfg == nullptr) return FP8MM_E_NULL;
  if (a->A == nullptr || a->B == nullptr || a->As == nullptr || a->Bs == nullptr || a->C == nullptr)
    return FP8MM_E_NULL;
  Geometry g;
  int rc = make_geometry(a->M, a->N, a->K, cfg, &g);
  if (rc != FP8MM_OK) return rc;
  if ((reinterpret_cast<uintptr_t>(a->A) & 15) || (reinterpret_cast<uintptr_t>(a->B) & 15) ||
      (reinterpret_cast<uintptr_t>(a->C) & 15) || a->ldc < a->N || (a->ldc % 8) != 0)
    return FP8MM_E_ALIGN;
  const size_t need = kStatusBytes + g.counter_bytes + g.partial_bytes;
  if (g.split > 1 && !g.cluster && (workspace == nullptr || ws_bytes < need)) return FP8MM_E_WORKSPACE;
  if (workspace != nullptr && ws_bytes < kStatusBytes) return FP8MM_E_WORKSPACE;

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FP8MM_E_DRIVER;
  if (g_dev[dev].sms == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
      return FP8MM_E_DRIVER;
    g_dev[dev].sms = sms;
  }

  if (g.gemv) {
    for (int d = 0; d < n_extra; ++d)
      if (extra_c[d] == nullptr) return FP8MM_E_NULL;
    return launch_gemv(dev, a, cfg, extra_c, n_extra, static_cast<cudaStream_t>(stream_));
  }

  CUtensorMap tm_tok, tm_wgt;
  rc = get_tensor_map(a->A, a->M, a->K, g.swap ? g.umma_n : (g.mx ? g.tt : 128), &tm_tok, g.kg);
  if (rc != FP8MM_OK) return rc;
  rc = get_tensor_map(a->B, a->N, a->K, (g.swap || g.pair) ? 128 : g.umma_n, &tm_wgt, g.kg, true);
  if (rc != FP8MM_OK) return rc;

  OutTargets outs;
  memset(&outs, 0, sizeof(outs));
  outs.n = 1 + n_extra;
  for (int d = 0; d < outs.n; ++d) {
    void* c = d == 0 ? a->C : extra_c[d - 1];
    if (c == nullptr) return FP8MM_E_NULL;
    if (reinterpret_cast<uintptr_t>(c) & 15) return FP8MM_E_ALIGN;
    outs.ptr[d] = static_cast<__nv_bfloat16*>(c);
    if (!g.swap) {
      rc = make_output_map(c, a->M, a->N, a->ldc, &outs.map[d], g.mx && g.tt == 256);
      if (rc != FP8MM_OK) return rc;
    }
  }

  unsigned char* ws = static_cast<unsigned char*>(workspace);
  KParams p;
  p.As = a->As;
  p.Bs = a->Bs;
  p.C = static_cast<__nv_bfloat16*>(a->C);
  p.status = reinterpret_cast<int*>(ws);
  // split-K scratch: needed by the workspace reduction, and handed to a cluster launch too when the
  // caller's workspace happens to be large enough, so that it can fall back if clusters have no room
  const size_t ws_path_need = kStatusBytes + kCounterBytes + (size_t)g.tiles * g.split * g.umma_n * 128 * sizeof(float);
  const bool ws_usable = g.split > 1 && ws != nullptr && ws_bytes >= ws_path_need;
  p.ws_counter = ws_usable ? reinterpret_cast<int*>(ws + kStatusBytes) : nullptr;
  p.ws_partial = ws_usable ? reinterpret_cast<float*>(ws + kStatusBytes + kCounterBytes) : nullptr;
  p.as_sm = a->as_stride_m;
  p.as_sk = a->as_stride_k;
  p.bs_sn = a->bs_stride_n;
  p.bs_sk = a->bs_stride_k;
  p.ldc = a->ldc;
  p.timeout_ns = timeout_ns();
  p.M = a->M;
  p.N = a->N;
  p.K = a->K;
  p.kb_per_unit = g.kbn;
  p.split = g.split;
  p.t_tiles = g.t_tiles;
  p.w_tiles = g.w_tiles;
  p.num_units = g.tiles * g.split;
  p.group_m = cfg->group_m;
  p.fd_split = make_fastdiv(g.split);
  p.fd_group = make_fastdiv(cfg->group_m * g.w_tiles);
  p.fd_gm = make_fastdiv(cfg->group_m);
  p.fd_tail = make_fastdiv(g.t_tiles % cfg->group_m);
  p.stages = g.stages;
  p.stg_slabs = g.stg_slabs;
  p.kg = g.kg;
  p.act_f32 = (cfg->flags & FP8MM_FLAG_ACT_SCALES_F32) ? 1 : 0;
  p.trace = nullptr;
#ifdef FP8MM_TRACE
  if (const char* e = getenv("FP8MM_TRACE_PTR")) p.trace = reinterpret_cast<long long*>(strtoull(e, nullptr, 0));
#endif

  // One CTA per SM unless the shared-memory footprint lets two share an SM.
  int per_sm = (int)((kMaxDynSmem + 1024) / (g.smem + 1024));
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 2) per_sm = 2;
  int grid = g_dev[dev].sms * per_sm;
  if (cfg->max_ctas > 0 && grid > cfg->max_ctas) grid = cfg->max_ctas;
  if (grid > p.num_units) grid = p.num_units;

  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (g.pair) {
    // one CTA pair per two SMs; the grid is a whole number of pairs
    int pairs = g_dev[dev].sms / 2;
    if (cfg->max_ctas > 0 && pairs > cfg->max_ctas / 2) pairs = cfg->max_ctas / 2 > 0 ? cfg->max_ctas / 2 : 1;
    if (pairs > p.num_units) pairs = p.num_units;
    return launch_plain(fp8mm_umma_2cta_kernel, 39, dev, g, tm_tok, tm_wgt, outs, p, 2 * pairs, stream);
  }
  if (g.mx && g.swap) {
    // slots 42..45 unsplit, 46..49 split-K through the workspace, 50..53 through a cluster
    PlainKernel kern[3] = {nullptr, nullptr, nullptr};
    int slot = 0;
    switch (g.tt) {
      case 16: kern[0] = fp8mm_mxs_kernel<16, 0>; kern[1] = fp8mm_mxs_kernel<16, 1>; kern[2] = fp8mm_mxs_kernel<16, 2>; slot = 42; break;
      case 32: kern[0] = fp8mm_mxs_kernel<32, 0>; kern[1] = fp8mm_mxs_kernel<32, 1>; kern[2] = fp8mm_mxs_kernel<32, 2>; slot = 43; break;
      case 64: kern[0] = fp8mm_mxs_kernel<64, 0>; kern[1] = fp8mm_mxs_kernel<64, 1>; kern[2] = fp8mm_mxs_kernel<64, 2>; slot = 44; break;
      case 128: kern[0] = fp8mm_mxs_kernel<128, 0>; kern[1] = fp8mm_mxs_kernel<128, 1>; kern[2] = fp8mm_mxs_kernel<128, 2>; slot = 45; break;
      default: return FP8MM_E_CONFIG;
    }
    if (g.split == 1 && g.kg == 2 && g.tt <= 64) {        // slots 54..56: the half-size form, two CTAs per SM
      PlainKernel k2 = g.tt == 16 ? fp8mm_mxs_kernel<16, 0, 2>
                                  : (g.tt == 32 ? fp8mm_mxs_kernel<32, 0, 2> : fp8mm_mxs_kernel<64, 0, 2>);
      return launch_plain(k2, slot + 12, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
    }
    if (g.split == 1) return launch_plain(kern[0], slot, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
    if (g.cluster) {
      // one CTA per unit, the `split` CTAs of a tile in one cluster; without room for such a cluster in this
      // context the workspace reduction gives the same bits, if the caller's workspace is large enough
      const int rc = launch_plain(kern[2], slot + 8, dev, g, tm_tok, tm_wgt, outs, p, p.num_units, stream, g.split);
      if (rc != kClusterUnschedulable) return rc;
      if (p.ws_partial == nullptr) return FP8MM_E_WORKSPACE;
    }
    return launch_plain(kern[1], slot + 4, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
  }
  if (g.mx) {
    return g.tt == 256 ? launch_plain(fp8mm_mx256_kernel, 41, dev, g, tm_tok, tm_wgt, outs, p, grid, stream)
                       : launch_plain(fp8mm_mx_kernel, 40, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
  }
  if (g.swap) {
    switch (g.umma_n) {
      case 16: return launch<16, true>(0, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
      case 32: return launch<32, true>(1, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
      case 64: return launch<64, true>(2, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
      case 128: return launch<128, true>(3, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
      case 256: return launch<256, true>(4, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
    }
  } else {
    switch (g.umma_n) {
      case 128: return launch<128, false>(5, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
      case 256: return launch<256, false>(6, dev, g, tm_tok, tm_wgt, outs, p, grid, stream);
    }
  }
  return FP8MM_E_CONFIG;
}

int fp8mm_b200_gemm(const fp8mm_args* a, const fp8mm_cfg* cfg, void* workspace, size_t ws_bytes,
                    void* stream) {
  return gemm_impl(a, cfg, workspace, ws_bytes, stream, nullptr, 0);
}

int fp8mm_b200_gemm_bcast(const fp8mm_args* a, const fp8mm_cfg* cfg, void* workspace, size_t ws_bytes,
                          void* stream, void* const* extra_c, int32_t n_extra) {
  return gemm_impl(a, cfg, workspace, ws_bytes, stream, extra_c, n_extra);
}

// ----------------------------------------------------- allocation-free entry point
size_t fp8mm_b200_static_scratch_bytes(void) { return kStaticScratchBytes; }

// Device address of the built-in scratch on the current device (looked up once per device).
static int static_scratch_address(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= fp8mm::kMaxDevices) return FP8MM_E_DRIVER;
  std::lock_guard<std::mutex> lk(fp8mm::g_mu);
  if (g_static_scratch_addr[dev] == nullptr) {
    // once per device, with that device current: symbol -> device address
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return FP8MM_E_DRIVER;
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return FP8MM_OK;
}

int fp8mm_b200_gemm_static_scratch(const fp8mm_args* args, const fp8mm_cfg* cfg, void* stream) {
  if (args == nullptr || cfg == nullptr) return FP8MM_E_NULL;
  const size_t need = fp8mm_b200_workspace_bytes(args->M, args->N, args->K, cfg);
  if (need == 0) return fp8mm_b200_validate(args->M, args->N, args->K, cfg);
  if (need > kStaticScratchBytes) return FP8MM_E_TOO_LARGE;
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != FP8MM_OK) return rc;
  // The tile counters must start at zero whatever the previous call left behind.  The status word in
  // front of them is NOT cleared here: a timeout recorded by an earlier call stays readable
  // (fp8mm_b200_static_scratch_status) until the caller has fetched it.
  if (cudaMemsetAsync(static_cast<unsigned char*>(scratch) + kStatusBytes, 0, kCounterBytes,
                      static_cast<cudaStream_t>(stream)) != cudaSuccess)
    return FP8MM_E_DRIVER;
  return fp8mm_b200_gemm(args, cfg, scratch, kStaticScratchBytes, stream);
}

int fp8mm_b200_static_scratch_status(int32_t* detail) {
  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc != FP8MM_OK) return rc;
  int32_t v = 0;
  if (cudaMemcpy(&v, scratch, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return FP8MM_E_DRIVER;
  if (detail != nullptr) *detail = v;
  if (v != 0 && cudaMemset(scratch, 0, sizeof(v)) != cudaSuccess) return FP8MM_E_DRIVER;   // fetched: start over
  return v == 0 ? FP8MM_OK : FP8MM_E_DEVICE_TIMEOUT;
}

}  // extern "C"
