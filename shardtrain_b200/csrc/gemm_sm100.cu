// Host launcher of the tcgen05 GEMM: builds the TMA tensor maps and picks the tile width.
#include <algorithm>
#include <array>
#include <atomic>
#include <mutex>
#include <unordered_map>

#include "api.h"
#include "gemm_sm100.cuh"

namespace stb {

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

}  // namespace

// Row-major bf16 matrix [rows, cols] with leading dimension ld -> 2-D tensor map whose box is
// box_cols x box_rows with 128-byte swizzle (box_cols * 2 bytes must be 128).
namespace {

// A tensor map is a pure function of (base, shape, pitch, box); the training loop presents the
// same few hundred operand descriptions every step (persistent weight buffers, allocator-stable
// activations), so encoded maps are memoised instead of calling the driver twice per GEMM.
struct MapKey {
  std::array<int64_t, 6> v;
  bool operator==(const MapKey& o) const { return v == o.v; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 0x9e3779b97f4a7c15ull;
    for (int64_t x : k.v) h = (h ^ static_cast<uint64_t>(x)) * 0x100000001b3ull + (h >> 29);
    return static_cast<size_t>(h);
  }
};
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;
constexpr size_t kMapCacheLimit = 8192;

}  // namespace

namespace {

enum MapKind { kMapBf16 = 0, kMapF32 = 1, kMapBf16Swizzle64 = 2 };

bool make_tensor_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld,
                     int box_cols, int box_rows, MapKind kind) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return false;
  const bool fp32 = kind == kMapF32;
  const int64_t esize = fp32 ? 4 : 2;
  const MapKey key{{static_cast<int64_t>(reinterpret_cast<uintptr_t>(base)), rows, cols, ld,
                    box_cols, box_rows + (static_cast<int64_t>(kind) << 20)}};
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) {
      *map = it->second;
      return true;
    }
  }
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld * esize)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  kind == kMapBf16Swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> lock(g_map_mutex);
  if (g_map_cache.size() >= kMapCacheLimit) g_map_cache.clear();
  g_map_cache.emplace(key, *map);
  return true;
}

}  // namespace

bool make_bf16_tensor_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols,
                          int64_t ld, int box_cols, int box_rows) {
  return make_tensor_map(map, base, rows, cols, ld, box_cols, box_rows, kMapBf16);
}

// Map for staged epilogue stores of bf16 planes: boxes of 32 rows x 32 columns (64-byte rows,
// 64B swizzle).
bool make_bf16_store_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols,
                         int64_t ld) {
  return make_tensor_map(map, base, rows, cols, ld, 32, 32, kMapBf16Swizzle64);
}

namespace {
std::atomic<int64_t> g_launches{0};
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
void count_launches(int64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int64_t launches_total() { return g_launches.load(std::memory_order_relaxed); }

int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v < 1)
      v = 1;
    return v;
  }();
  return n;
}

namespace {

// How the tail wave of `tiles` tiles is cut along K (see GemmSplit).  `want`: 0 = rule, 1 = never,
// n > 1 = exactly n (tests).  Returns the split factor and fills full / kb_per.
int plan_split(int tiles, int num_kb, int want, int* full, int* kb_per) {
  const int sms = sm_count();
  *full = (tiles / sms) * sms;
  const int rem = tiles - *full;
  *kb_per = num_kb;
  if (rem == 0 || want == 1) return 1;
  // parking and re-reading a partial tile costs about as much as 10 k-blocks: only splits that
  // keep at least 32 k-blocks each pay off.  (Cutting the tiles of a GEMM smaller than half a
  // wave down to 6 k-blocks was tried and measured slower: 29 us against 23 us at
  // 512 x 2048 x 1536.)
  int split = want > 1 ? want : std::min({sms / rem, 8, num_kb / 32});
  split = std::min(split, sms / rem);
  if (split < 2) return 1;
  *kb_per = (num_kb + split - 1) / split;
  return (num_kb + *kb_per - 1) / *kb_per;      // no empty K range
}

// Partial-tile workspace and tile counters of the tail split, one set per (device, stream): two
// GEMMs can only overlap on different streams, and each stream then has its own set.
struct SplitBuffers {
  float* workspace = nullptr;
  int* counters = nullptr;
};
std::mutex g_split_mutex;
std::unordered_map<uint64_t, SplitBuffers> g_split_buffers;

cudaError_t split_buffers(cudaStream_t stream, SplitBuffers* out) {
  int dev = 0;
  cudaGetDevice(&dev);
  const uint64_t key = (static_cast<uint64_t>(dev) << 56) ^ reinterpret_cast<uint64_t>(stream);
  std::lock_guard<std::mutex> lock(g_split_mutex);
  auto it = g_split_buffers.find(key);
  if (it == g_split_buffers.end()) {
    SplitBuffers b;
    const size_t units = static_cast<size_t>(sm_count());
    cudaError_t e = cudaMalloc(&b.workspace, units * kGemmBM * 256 * sizeof(float));
    if (e != cudaSuccess) return e;
    e = cudaMalloc(&b.counters, units * sizeof(int));
    if (e != cudaSuccess) return e;
    // ordered on the launching stream: the first kernel that uses the counters runs there
    e = cudaMemsetAsync(b.counters, 0, units * sizeof(int), stream);
    if (e != cudaSuccess) return e;
    it = g_split_buffers.emplace(key, b).first;
  }
  *out = it->second;
  return cudaSuccess;
}

// Arrival flags of the PULL variant, one buffer per (device, stream), and the epoch counter that
// makes every launch's flag value unique (flags are never cleared).
constexpr int kPullFlagCount = 65536;       // 8-row groups: up to 524288 rows of A
std::unordered_map<uint64_t, uint32_t*> g_pull_flags;
uint32_t g_pull_epoch = 0;

cudaError_t pull_flags(cudaStream_t stream, uint32_t** flags, uint32_t* epoch) {
  int dev = 0;
  cudaGetDevice(&dev);
  const uint64_t key = (static_cast<uint64_t>(dev) << 56) ^ reinterpret_cast<uint64_t>(stream);
  std::lock_guard<std::mutex> lock(g_split_mutex);
  auto it = g_pull_flags.find(key);
  if (it == g_pull_flags.end()) {
    uint32_t* p = nullptr;
    cudaError_t e = cudaMalloc(&p, kPullFlagCount * sizeof(uint32_t));
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(p, 0, kPullFlagCount * sizeof(uint32_t), stream);
    if (e != cudaSuccess) return e;
    it = g_pull_flags.emplace(key, p).first;
  }
  *flags = it->second;
  if (++g_pull_epoch == 0) ++g_pull_epoch;   // 0 is the cleared state
  *epoch = g_pull_epoch;
  return cudaSuccess;
}

template <int BN, bool A_MN, bool B_MN>
cudaError_t launch_variant(const GemmCall& c, int* status, cudaStream_t stream) {
  CUtensorMap ta, tb;
  bool ok;
  if (!A_MN)
    ok = make_bf16_tensor_map(&ta, c.a, c.M, c.K, c.lda, 64, kGemmBM);
  else
    ok = make_bf16_tensor_map(&ta, c.a, c.K, c.M, c.lda, 64, 64);
  if (!B_MN)
    ok = ok && make_bf16_tensor_map(&tb, c.b, c.N, c.K, c.ldb, 64, c.gated_inter > 0 ? BN / 2 : BN);
  else
    ok = ok && make_bf16_tensor_map(&tb, c.b, c.K, c.N, c.ldb, 64, 64);
  if (!ok) return cudaErrorInvalidValue;

  GemmEpilogue ep;
  ep.out = c.out;
  ep.bias = c.bias;
  ep.residual = c.residual;
  ep.mul = nullptr;
  ep.ldo = c.ldo;
  ep.out_fp32 = c.out_fp32 ? 1 : 0;
  ep.accumulate = c.accumulate ? 1 : 0;
  ep.alpha = c.alpha;
  ep.gated_out = c.gated_out;
  ep.gated_inter = c.gated_inter > 0 ? c.gated_inter : 0;
  ep.scatter_degree = c.scatter_degree > 1 ? c.scatter_degree : 0;
  ep.scatter_seq = c.scatter_seq;
  ep.scatter_seq_local = c.scatter_seq_local;
  ep.scatter_broadcast = c.scatter_broadcast ? 1 : 0;
  for (int i = 0; i < 8; ++i) ep.scatter_out[i] = i < ep.scatter_degree ? c.scatter_out[i] : nullptr;
  // Plain outputs leave through TMA stores of 32 x 128-byte boxes (32 fp32 or 64 bf16 columns).
  // `staged_store` = -1 in the call keeps the per-thread row stores (tests compare the two).
  // The SwiGLU epilogue stores 32-column boxes (64-byte rows, 64B swizzle) of three planes: the
  // gate half and the up half of `out` (a map each, so that a box at the ragged end of the gate
  // half cannot spill into the up half) and `gated_out`.
  CUtensorMap tc = ta, tc_up = ta, tc_h = ta;
  ep.staged_store = 0;
  if (c.staged_store >= 0 && ep.scatter_degree == 0 && !c.accumulate &&
      (c.ldo * (c.out_fp32 ? 4 : 2)) % 16 == 0) {
    bool made;
    if (ep.gated_inter > 0) {
      const __nv_bfloat16* gu = reinterpret_cast<const __nv_bfloat16*>(c.out);
      made = make_tensor_map(&tc, gu, c.M, ep.gated_inter, c.ldo, 32, 32, kMapBf16Swizzle64) &&
             make_tensor_map(&tc_up, gu + ep.gated_inter, c.M, ep.gated_inter, c.ldo, 32, 32,
                             kMapBf16Swizzle64) &&
             make_tensor_map(&tc_h, c.gated_out, c.M, ep.gated_inter, ep.gated_inter, 32, 32,
                             kMapBf16Swizzle64);
    } else {
      made = make_tensor_map(&tc, c.out, c.M, c.N, c.ldo, c.out_fp32 ? 32 : 64, 32,
                             c.out_fp32 ? kMapF32 : kMapBf16);
    }
    if (made)
      ep.staged_store = 1;
    else
      tc = tc_up = tc_h = ta;
  }

  constexpr int smem = GemmSmem<BN>::kTotal;
  const int m_tiles = (c.M + kGemmBM - 1) / kGemmBM;
  const int n_tiles = c.gated_inter > 0 ? (c.gated_inter + BN / 2 - 1) / (BN / 2) : (c.N + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;
  const int num_kb = (c.K + kGemmBK - 1) / kGemmBK;
  GemmSplit sp{};
  sp.split = plan_split(tiles, num_kb, c.gated_inter > 0 ? 1 : c.split_k, &sp.full_tiles,
                        &sp.kb_per_split);
  if (sp.split > 1) {
    SplitBuffers buffers;
    const cudaError_t e = split_buffers(stream, &buffers);
    if (e != cudaSuccess) return e;
    sp.workspace = buffers.workspace;
    sp.counters = buffers.counters;
  } else {
    sp.full_tiles = tiles;
  }
  sp.total_units = sp.full_tiles + (tiles - sp.full_tiles) * sp.split;
  const int grid = std::min(sp.total_units, sm_count());   // persistent: one CTA per SM
  if constexpr (!A_MN) {
    if (c.pull_degree > 1) {
      GemmPull pull{};
      for (int i = 0; i < c.pull_degree; ++i) pull.peers[i] = c.pull_peers[i];
      pull.degree = c.pull_degree;
      pull.batch = c.pull_batch;
      pull.seq_local = c.pull_seq_local;
      pull.src_ld = c.pull_src_ld;
      pull.dst = const_cast<void*>(c.a);
      pull.dst_ld = c.lda;
      const cudaError_t e = pull_flags(stream, &pull.flags, &pull.epoch);
      if (e != cudaSuccess) return e;
      auto kernel = gemm_pull_bf16_tcgen05_kernel<BN, B_MN>;
      static std::once_flag once;
      static cudaError_t attr_err = cudaSuccess;
      std::call_once(once, [&] {
        attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      });
      if (attr_err != cudaSuccess) return attr_err;
      kernel<<<grid, kGemmThreads + kPullThreads, smem, stream>>>(ta, tb, tc, tc_up, tc_h, ep, sp,
                                                                 pull, c.M, c.N, c.K, status);
      count_launch();
      return cudaGetLastError();
    }
  }
  auto kernel = gemm_bf16_tcgen05_kernel<BN, A_MN, B_MN>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  });
  if (attr_err != cudaSuccess) return attr_err;
  kernel<<<grid, kGemmThreads, smem, stream>>>(ta, tb, tc, tc_up, tc_h, ep, sp, c.M, c.N, c.K,
                                               status);
  count_launch();
  return cudaGetLastError();
}

template <int BN>
cudaError_t dispatch_major(const GemmCall& c, int* status, cudaStream_t stream) {
  if (!c.a_mn && !c.b_mn) return launch_variant<BN, false, false>(c, status, stream);
  if (!c.a_mn && c.b_mn) return launch_variant<BN, false, true>(c, status, stream);
  if (c.a_mn && c.b_mn) return launch_variant<BN, true, true>(c, status, stream);
  return launch_variant<BN, true, false>(c, status, stream);
}

}  // namespace

cudaError_t launch_gemm_bf16(const GemmCall& c, int* status, cudaStream_t stream) {
  if (c.M <= 0 || c.N <= 0 || c.K <= 0) return cudaErrorInvalidValue;
  // TMA needs 16-byte aligned bases and strides; the vectorised epilogue needs N % 8 == 0.
  auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!aligned16(c.a) || !aligned16(c.b) || !aligned16(c.out) || (c.lda % 8) || (c.ldb % 8) ||
      (c.N % 8) || (c.ldo % (c.out_fp32 ? 4 : 8)))
    return cudaErrorInvalidValue;
  if (c.residual != nullptr && !aligned16(c.residual)) return cudaErrorInvalidValue;
  if (c.accumulate && !c.out_fp32) return cudaErrorInvalidValue;
  if (c.scatter_degree > 1) {
    // the scatter epilogue writes fp32 rows; every destination must be 16-byte aligned and the
    // sequence must split evenly over the owners
    if (!c.out_fp32 || c.accumulate || c.residual != nullptr || c.bias != nullptr ||
        c.scatter_degree > 8 ||
        (!c.scatter_broadcast &&
         (c.scatter_seq_local <= 0 || c.scatter_seq != c.scatter_seq_local * c.scatter_degree ||
          c.M % c.scatter_seq)))
      return cudaErrorInvalidValue;
    for (int i = 0; i < c.scatter_degree; ++i)
      if (c.scatter_out[i] == nullptr || !aligned16(c.scatter_out[i])) return cudaErrorInvalidValue;
  }
  if (c.pull_degree > 1) {
    // A is gathered inside the GEMM: K-major A only, whole 16-byte pieces per row, aligned peers
    if (c.a_mn || c.pull_degree > 8 || c.pull_batch <= 0 || c.pull_seq_local <= 0 || (c.K % 8) ||
        (c.pull_src_ld % 8) ||
        static_cast<int64_t>(c.pull_batch) * c.pull_degree * c.pull_seq_local != c.M ||
        (c.M + kPullRows - 1) / kPullRows > kPullFlagCount)
      return cudaErrorInvalidValue;
    for (int i = 0; i < c.pull_degree; ++i)
      if (c.pull_peers[i] == nullptr || !aligned16(c.pull_peers[i])) return cudaErrorInvalidValue;
  }
  if (c.gated_inter > 0) {
    // SwiGLU epilogue: 256-wide tiles (128 gate + 128 up columns), forward operand order, bf16
    if (c.a_mn || c.b_mn || c.out_fp32 || c.accumulate || c.bias != nullptr ||
        c.residual != nullptr || c.scatter_degree > 1 || c.gated_out == nullptr ||
        !aligned16(c.gated_out) || c.N != 2 * c.gated_inter || c.gated_inter % 8)
      return cudaErrorInvalidValue;
    return dispatch_major<256>(c, status, stream);
  }
  int bn = c.force_bn;
  if (bn == 0) {
    // Persistent kernel, one CTA per SM: the run time is (waves of tiles) x (time of one tile).
    // Measured on B200, a k-block of a 128 x BN tile is bound by the shared-memory operand reads
    // of the MMAs, i.e. its time goes with 128 + BN, not with BN; the tail wave counts 1/split
    // when its tiles are cut along K.  Pick the width with the smallest product.
    const int sms = sm_count();
    const int m_tiles = (c.M + kGemmBM - 1) / kGemmBM;
    const int num_kb = (c.K + kGemmBK - 1) / kGemmBK;
    double best = -1.0;
    for (int cand : {256, 192, 128}) {
      const int tiles = m_tiles * ((c.N + cand - 1) / cand);
      int full, kb_per;
      const int split = plan_split(tiles, num_kb, c.split_k, &full, &kb_per);
      // whole waves + the tail wave (shortened by its K split, plus the cost of parking and
      // re-reading the partial tiles)
      double waves = full / sms;
      if (tiles > full) waves += 1.0 / split + (split > 1 ? 0.06 : 0.0);
      const double cost = waves * (kGemmBM + cand);
      if (best < 0 || cost < best) {
        best = cost;
        bn = cand;
      }
    }
  }
  if (bn == 256) return dispatch_major<256>(c, status, stream);
  if (bn == 192) return dispatch_major<192>(c, status, stream);
  if (bn == 128) return dispatch_major<128>(c, status, stream);
  return cudaErrorInvalidValue;
}

}  // namespace stb
