// Parameter all-gather fused into the GEMM that consumes the parameters (sm_100a).
//
//   out[M, N] = A[M, K] * W[N, K]^T (+ bias)          or, gated: gu = A * W_gu^T, h = silu(g) * u
//
// W is not a local matrix: it is the concatenation of up to four FSDP-sharded parameters (q|k|v,
// gate|up) whose flat shards live in the F ranks' shard arenas.  The reference materialises them
// with `all_gather_into_tensor` + copy-out and then calls F.linear
// (src/sharded_runtime/runtime/materializer.py:31-114, src/sharded_runtime/runtime/layout.py:77-90,
// src/sharded_runtime/runtime/qwen2_operators.py:50-64).  Here one kernel does both:
//
//   * a CTA owns one tile of BN weight rows and walks K once ("weight stationary");
//   * four producer warps pull that tile's rows straight out of the owning ranks' arenas with
//     16-byte cp.async copies (plain peer loads through NVSwitch; several stages in flight per
//     thread) into the 128-byte-swizzled stage buffers the tensor core reads, and copy what they
//     pulled into the unit's local full-parameter buffer as a by-product (later consumers of the
//     same parameters -- a second pass over M, the backward of a retained unit -- read it locally);
//   * the activation A (a few hundred rows, L2 resident) arrives by TMA from local memory;
//   * up to 512 / BN accumulators of 128 x BN live in TMEM at once, one per 128-row tile of A, so
//     for M <= 128 * (512 / BN) every weight byte crosses NVLink exactly once and is never read
//     back from HBM for this GEMM.  For larger M the remaining row tiles are further passes whose
//     weight operand comes from the local buffer the first pass filled.
//
// Tensor maps cover local memory only; no load uses cluster multicast; no wait is unbounded.
// CTA = 6 warps: warp 0 issues the TMA loads of A, warp 1 owns TMEM and issues the MMAs, warps
// 2..5 are the weight producers and, after the last k-block, the epilogue.
#include <algorithm>
#include <mutex>

#include "api.h"
#include "common.cuh"

namespace stb {

bool make_bf16_tensor_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols,
                          int64_t ld, int box_cols, int box_rows);
bool make_bf16_store_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld);

namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kThreads = 192;
constexpr int kProducers = 128;
constexpr int kAStages = 8;          // two k-blocks of four row tiles: hides the L2 latency of A
constexpr int kLag = 3;              // weight stages a producer keeps in flight before it waits
constexpr int kATile = kBM * kBK * 2;

template <int BN>
struct AgSmem {
  static constexpr int kBTile = BN * kBK * 2;
  static constexpr int kBStages = BN == 128 ? 5 : 8;
  static constexpr int kBarrierBytes = 512;
  static constexpr int kTotal = kBStages * kBTile + kAStages * kATile + 1024 + kBarrierBytes;
  static_assert(kBStages * kBTile >= 4 * 12288, "the epilogue stages 12 KB per warp in the weight stages");
};

struct AgParams {
  AgWeights w;
  void* out;              // bf16 [M, ldo]
  const float* bias;      // optional fp32 [N]
  void* gated_out;        // bf16 [M, gated_inter] (gated mode)
  int64_t ldo;
  int gated_inter;        // > 0: W = gate|up, a tile holds BN/2 gate rows and the matching up rows
  int M, N, K;
  int mt;                 // row tiles of A per pass (accumulators alive in TMEM)
  int* status;
  // Staged epilogue: 32 x 32 bf16 boxes leave through TMA stores from shared memory (the weight
  // stages, which are idle once a pass's MMAs have completed).  Plain mode uses `map_out`; gated
  // mode one map per plane (gate half, up half, product).
  int staged;
  CUtensorMap map_out, map_up, map_h;
};

__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Segment table as the producers use it (copied to shared memory once per CTA: indexing the
// kernel parameters with a run-time index would spill them to local memory).
struct SegShared {
  int64_t q;          // shard length of the parameter
  int64_t shard_off;  // element offset of the parameter's shard inside every rank's arena
  int64_t full_off;   // element offset of the parameter inside the local full buffer
  int first_row;      // first row of the parameter inside the fused weight
  int rows;
  int vec;            // 16-byte copies are safe (alignment; 8 elements never straddle a rank)
  int pad;
};

// Where one row of a weight tile comes from: parameter `seg`, flat element index of (row, k = 0)
// inside that parameter; seg < 0 marks a row beyond the weight (zero filled).
struct RowSource {
  uint32_t flat0;     // < 2^31: the host rejects larger parameters
  int seg;
};

__device__ __forceinline__ RowSource locate_row(const SegShared* segs, int n_segs, int fused_row,
                                                int n_rows, int K) {
  RowSource r{0, -1};
  if (fused_row < 0 || fused_row >= n_rows) return r;
  for (int j = 0; j < n_segs; ++j) {
    if (fused_row < segs[j].first_row + segs[j].rows) {
      r.flat0 = static_cast<uint32_t>(fused_row - segs[j].first_row) * static_cast<uint32_t>(K);
      r.seg = j;
      return r;
    }
  }
  return r;
}

// One 16-byte chunk of a weight stage by the general route: rows beyond the weight and the K
// tail are zero filled; later passes read the local full buffer; otherwise the eight elements are
// fetched from their owners (fp32 or bf16 arenas), one by one where a 16-byte piece could straddle
// two owners or be misaligned.  Kept out of line: the common case never comes here.
__device__ __noinline__ void copy_chunk_general(const AgParams& p, const SegShared* segs,
                                                RowSource rs, uint8_t* dst, int k0, bool from_peers) {
  __nv_bfloat16 v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = __float2bfloat16(0.f);
  if (rs.seg >= 0 && k0 < p.K) {
    const SegShared& sg = segs[rs.seg];
    const uint32_t flat = rs.flat0 + static_cast<uint32_t>(k0);
    const uint32_t q32 = static_cast<uint32_t>(sg.q);
    const bool whole = sg.vec && k0 + 8 <= p.K;
    if (!from_peers) {
      const __nv_bfloat16* g = p.w.full + sg.full_off + flat;
      for (int e = 0; e < 8 && k0 + e < p.K; ++e) v[e] = g[e];
    } else if (whole && p.w.shadow[0] == nullptr && flat / q32 == (flat + 7) / q32) {
      const uint32_t owner = flat / q32;
      const float4* g = reinterpret_cast<const float4*>(p.w.shard[owner] + sg.shard_off +
                                                        (flat - owner * q32));
      const float4 lo = g[0], hi = g[1];
      v[0] = __float2bfloat16(lo.x); v[1] = __float2bfloat16(lo.y);
      v[2] = __float2bfloat16(lo.z); v[3] = __float2bfloat16(lo.w);
      v[4] = __float2bfloat16(hi.x); v[5] = __float2bfloat16(hi.y);
      v[6] = __float2bfloat16(hi.z); v[7] = __float2bfloat16(hi.w);
    } else {
      for (int e = 0; e < 8 && k0 + e < p.K; ++e) {
        const uint32_t f = flat + e;
        const uint32_t owner = f / q32;
        const int64_t off = sg.shard_off + (f - owner * q32);
        v[e] = p.w.shadow[0] != nullptr ? p.w.shadow[owner][off]
                                        : __float2bfloat16(p.w.shard[owner][off]);
      }
    }
  }
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(v);
}

// Mirror one landed chunk into the local full buffer, element by element where needed.
__device__ __noinline__ void mirror_chunk_general(const AgParams& p, const SegShared* segs,
                                                  RowSource rs, const uint8_t* chunk_smem, int k0) {
  if (rs.seg < 0 || k0 >= p.K) return;
  const SegShared& sg = segs[rs.seg];
  const uint4 x = *reinterpret_cast<const uint4*>(chunk_smem);
  __nv_bfloat16* g = p.w.full + sg.full_off + rs.flat0 + k0;
  if (sg.vec && k0 + 8 <= p.K) {
    *reinterpret_cast<uint4*>(g) = x;
  } else {
    const __nv_bfloat16* xv = reinterpret_cast<const __nv_bfloat16*>(&x);
    for (int e = 0; e < 8 && k0 + e < p.K; ++e) g[e] = xv[e];
  }
}

// Every CTA reads the whole of A, one k-block after the other.  If all CTAs walked K in the same
// order they would ask the L2 for the same few lines at the same moment; each tile therefore
// starts at its own k-block and wraps around (the sum over K does not depend on the order up to
// fp32 rounding).
__device__ __forceinline__ int k_rotation(int tile, int num_kb) { return (tile * 7) % num_kb; }

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_allgather_kernel(const __grid_constant__ CUtensorMap tma_a,
                      const __grid_constant__ AgParams p) {
  using S = AgSmem<BN>;
  constexpr int NB = S::kBStages;
  if (kernel_should_skip(p.status)) return;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* b_tiles = smem;
  uint8_t* a_tiles = smem + NB * S::kBTile;
  uint64_t* b_full = reinterpret_cast<uint64_t*>(a_tiles + kAStages * kATile);
  uint64_t* b_empty = b_full + NB;
  uint64_t* a_full = b_empty + NB;
  uint64_t* a_empty = a_full + kAStages;
  uint64_t* acc_full = a_empty + kAStages;     // [1]
  uint64_t* acc_empty = acc_full + 1;          // [1], 128 arrivals
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);
  SegShared* segs = reinterpret_cast<SegShared*>(tmem_ptr + 4);   // 4 x 40 bytes, 16-byte aligned

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool gated = p.gated_inter > 0;
  const int tile_cols = gated ? BN / 2 : BN;
  const int n_span = gated ? p.gated_inter : p.N;
  const int n_tiles = (n_span + tile_cols - 1) / tile_cols;
  const int m_tiles = (p.M + kBM - 1) / kBM;
  const int passes = (m_tiles + p.mt - 1) / p.mt;
  const int num_kb = (p.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NB; ++s) {
      mbar_init(&b_full[s], kProducers);
      mbar_init(&b_empty[s], 1);
    }
    for (int s = 0; s < kAStages; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&a_empty[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, kProducers);
    *abort_flag = 0;
    int first = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const AgSegment sg = p.w.seg[j];
      const bool used = j < p.w.n_segs;
      segs[j].q = used ? sg.q : 1;
      segs[j].shard_off = sg.shard_off;
      segs[j].full_off = sg.full_off;
      segs[j].first_row = first;
      segs[j].rows = used ? sg.rows : 0;
      segs[j].vec = (sg.q % 8 == 0) && (sg.shard_off % 8 == 0) && (sg.full_off % 8 == 0) &&
                    (p.K % 8 == 0);
      first += segs[j].rows;
    }
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&tma_a);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ A: TMA from local memory
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int rot = k_rotation(tile, num_kb);
        for (int pass = 0; pass < passes && ok; ++pass) {
          const int m_first = pass * p.mt;
          const int m_count = min(p.mt, m_tiles - m_first);
          for (int step = 0; step < num_kb && ok; ++step) {
            const int kb = (step + rot) % num_kb;
            for (int m = 0; m < m_count; ++m, ++it) {
              const int s = it % kAStages;
              if (!mbar_wait(&a_empty[s], ((it / kAStages) & 1) ^ 1, p.status,
                             kErrProducerEmptyWait)) {
                *abort_flag = 1;
                ok = false;
                break;
              }
              mbar_expect_tx(&a_full[s], kATile);
              tma_load_2d(a_tiles + s * kATile, &tma_a, &a_full[s], kb * kBK, (m_first + m) * kBM);
            }
          }
        }
      }
      if (*abort_flag) {   // error path only: drain the copies nobody consumed
        for (int k = max(0, it - kAStages); k < it; ++k)
          mbar_wait(&a_full[k % kAStages], (k / kAStages) & 1, p.status, kErrDrainWait);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, false, false);
      int ita = 0, itb = 0, round = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        for (int pass = 0; pass < passes && ok; ++pass, ++round) {
          const int m_count = min(p.mt, m_tiles - pass * p.mt);
          // the epilogue of the previous round must have drained the accumulators
          if (!mbar_wait(acc_empty, (round & 1) ^ 1, p.status, kErrMmaFullWait)) {
            *abort_flag = 1;
            break;
          }
          tc_fence_after_sync();
          for (int kb = 0; kb < num_kb && ok; ++kb, ++itb) {
            const int sb = itb % NB;
            if (!mbar_wait(&b_full[sb], (itb / NB) & 1, p.status, kErrMmaFullWait)) {
              *abort_flag = 1;
              ok = false;
              break;
            }
            const uint32_t b_base = smem_u32(b_tiles + sb * S::kBTile);
            for (int m = 0; m < m_count; ++m, ++ita) {
              const int sa = ita % kAStages;
              if (!mbar_wait(&a_full[sa], (ita / kAStages) & 1, p.status, kErrMmaFullWait)) {
                *abort_flag = 1;
                ok = false;
                break;
              }
              tc_fence_after_sync();
              const uint32_t a_base = smem_u32(a_tiles + sa * kATile);
#pragma unroll
              for (int k = 0; k < kBK / 16; ++k) {
                const uint64_t da = make_smem_desc_sw128(a_base + k * 32, 16, 1024);
                const uint64_t db = make_smem_desc_sw128(b_base + k * 32, 16, 1024);
                tc_mma_f16(tmem_base + m * BN, da, db, idesc, (kb | k) != 0 ? 1u : 0u);   // kb: step
              }
              tc_commit(&a_empty[sa]);
            }
            if (ok) tc_commit(&b_empty[sb]);   // the weight stage is free once these MMAs read it
          }
          if (ok) tc_commit(acc_full);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ weight producers, then epilogue
    const int t = threadIdx.x - 64;          // 0..127
    const int chunk = t & 7;                 // 16-byte chunk of the 128-byte row segment
    constexpr int ROWS_PER_THREAD = BN / 16; // rows t/8, t/8 + 16, ...
    const int q4 = warp & 3;                 // TMEM lane quarter this warp may read
    const int row_in_tile = q4 * 32 + lane;  // accumulator row of this thread in the epilogue
    int itb = 0, round = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      const int n0 = tile * tile_cols;
      const int rot = k_rotation(tile, num_kb);
      RowSource src[ROWS_PER_THREAD];
      uint32_t row_off[ROWS_PER_THREAD];     // byte offset of this thread's chunk inside a stage
#pragma unroll
      for (int i = 0; i < ROWS_PER_THREAD; ++i) {
        const int r = (t >> 3) + i * 16;     // row inside the tile
        int fused_row;
        if (gated) {
          // first half of the tile: gate rows n0.., second half: the up rows of the same indices
          const int idx = n0 + (r < BN / 2 ? r : r - BN / 2);
          fused_row = idx >= p.gated_inter ? -1 : (r < BN / 2 ? idx : p.gated_inter + idx);
        } else {
          fused_row = n0 + r;
        }
        src[i] = locate_row(segs, p.w.n_segs, fused_row, p.N, p.K);
        row_off[i] = static_cast<uint32_t>(r * 128 + ((chunk ^ (r & 7)) << 4));
      }
      for (int pass = 0; pass < passes; ++pass, ++round) {
        const bool from_peers = pass == 0;
        const bool mirror = from_peers && p.w.full != nullptr;
        // Per row, resolved once per pass: where the row's chunks are read from when the whole row
        // sits in one place (one owner's bf16 shard, or the local full buffer on later passes)
        // and 16-byte pieces are safe, and where they are mirrored to.  The per-stage loop is then
        // a handful of instructions per chunk; anything else (fp32 on the wire, rows that
        // straddle two owners, unaligned shards, the K tail) goes through copy_chunk_general.
        const __nv_bfloat16* fast_src[ROWS_PER_THREAD];
        __nv_bfloat16* mirror_dst[ROWS_PER_THREAD];
#pragma unroll
        for (int i = 0; i < ROWS_PER_THREAD; ++i) {
          fast_src[i] = nullptr;
          mirror_dst[i] = nullptr;
          if (src[i].seg < 0) continue;
          const SegShared& sg = segs[src[i].seg];
          if (!sg.vec) continue;
          if (mirror) mirror_dst[i] = p.w.full + sg.full_off + src[i].flat0;
          if (!from_peers) {
            fast_src[i] = p.w.full + sg.full_off + src[i].flat0;
          } else if (p.w.shadow[0] != nullptr) {
            const uint32_t q32 = static_cast<uint32_t>(sg.q);
            const uint32_t owner = src[i].flat0 / q32;
            if ((src[i].flat0 + static_cast<uint32_t>(p.K) - 1) / q32 == owner)
              fast_src[i] = p.w.shadow[owner] + sg.shard_off + (src[i].flat0 - owner * q32);
          }
        }
        // The copies of weight stage `done` (k-block `done_kb` of this pass) have landed for this
        // thread: mirror its chunks into the local full buffer, then hand the stage to the MMAs.
        auto publish = [&](int done, int done_kb) {
          if (mirror) {
            const uint8_t* st = b_tiles + (done % NB) * S::kBTile;
            const int dk0 = done_kb * kBK + chunk * 8;
            if (dk0 + 8 <= p.K) {
#pragma unroll
              for (int i = 0; i < ROWS_PER_THREAD; ++i) {
                if (mirror_dst[i] != nullptr)
                  *reinterpret_cast<uint4*>(mirror_dst[i] + dk0) =
                      *reinterpret_cast<const uint4*>(st + row_off[i]);
                else
                  mirror_chunk_general(p, segs, src[i], st + row_off[i], dk0);
              }
            } else {
#pragma unroll
              for (int i = 0; i < ROWS_PER_THREAD; ++i)
                mirror_chunk_general(p, segs, src[i], st + row_off[i], dk0);
            }
          }
          fence_proxy_async();                 // generic-proxy writes -> visible to the tensor core
          mbar_arrive(&b_full[done % NB]);
        };
        // ---- produce the weight stages of this pass
        int waiting = 0;                      // stages issued whose copies were not yet awaited
        for (int step = 0; step < num_kb && ok; ++step, ++itb) {
          const int kb = (step + rot) % num_kb;
          const int sb = itb % NB;
          if (!mbar_wait(&b_empty[sb], ((itb / NB) & 1) ^ 1, p.status, kErrProducerEmptyWait)) {
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* stage = b_tiles + sb * S::kBTile;
          const uint32_t stage_addr = smem_u32(stage);
          const int k0 = kb * kBK + chunk * 8;
          if (k0 + 8 <= p.K) {
#pragma unroll
            for (int i = 0; i < ROWS_PER_THREAD; ++i) {
              if (fast_src[i] != nullptr)
                cp_async_16(stage_addr + row_off[i], fast_src[i] + k0);
              else
                copy_chunk_general(p, segs, src[i], stage + row_off[i], k0, from_peers);
            }
          } else {
#pragma unroll
            for (int i = 0; i < ROWS_PER_THREAD; ++i)
              copy_chunk_general(p, segs, src[i], stage + row_off[i], k0, from_peers);
          }
          cp_async_commit();
          ++waiting;
          if (waiting > kLag) {
            cp_async_wait<kLag>();               // the oldest outstanding stage is complete
            publish(itb - kLag, (step - kLag + rot) % num_kb);
            --waiting;
          }
        }
        // ---- tail: the stages still in flight
        cp_async_wait<0>();
        if (ok) {
          for (int back = waiting; back >= 1; --back)
            publish(itb - back, (num_kb - back + rot) % num_kb);
        }
        if (mirror && passes > 1) {
          // the next pass of this CTA reads back what these 128 threads just wrote to `full`
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }

        // ---- epilogue of this pass: m_count accumulators of 128 x BN
        const int m_first = pass * p.mt;
        const int m_count = min(p.mt, m_tiles - m_first);
        if (ok) ok = mbar_wait(acc_full, round & 1, p.status, kErrEpilogueAccumWait);
        tc_fence_after_sync();
        const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
        // Every MMA of this pass has completed (acc_full), so every thread's mirror reads of the
        // weight stages have too (a stage is handed over only after them): the stage memory is
        // free until the next pass and serves as the staging area, 12 KB per warp.
        const bool staged = p.staged != 0 && __all_sync(0xffffffffu, ok);
        uint8_t* stage_base = b_tiles + q4 * 12288;
        int issued = 0;
        for (int m = 0; m < m_count && ok; ++m) {
          const int64_t g_row = static_cast<int64_t>(m_first + m) * kBM + row_in_tile;
          const bool row_ok = g_row < p.M;
          const int band_row = (m_first + m) * kBM + q4 * 32;
          const uint32_t acc = tmem_base + lane_base + m * BN;
          if (gated) {
            __nv_bfloat16* gu_row = reinterpret_cast<__nv_bfloat16*>(p.out) + g_row * p.ldo;
            __nv_bfloat16* h_row = reinterpret_cast<__nv_bfloat16*>(p.gated_out) + g_row * p.gated_inter;
#pragma unroll 1
            for (int c = 0; c < BN / 64; ++c) {
              uint32_t rg[32], ru[32];
              tmem_ld_32x32(acc + c * 32, rg);
              tmem_ld_32x32(acc + BN / 2 + c * 32, ru);
              tmem_ld_wait();
              const int col0 = n0 + c * 32;
              if (staged ? (band_row >= p.M || col0 >= p.gated_inter)
                         : (!row_ok || col0 >= p.gated_inter))
                continue;
              // staged: two sets of three 2 KB boxes per warp, one bulk group per chunk
              uint8_t* slot = stage_base + (issued & 1) * 6144;
              if (staged) {
                if (lane == 0) bulk_wait_group_read<1>();
                __syncwarp();
              }
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                if (!staged && col0 + i >= p.gated_inter) break;
                uint4 pg, pu, ph;
                uint32_t* wg = &pg.x;
                uint32_t* wu = &pu.x;
                uint32_t* wh = &ph.x;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  wg[j] = pack_bf16x2(__uint_as_float(rg[i + 2 * j]), __uint_as_float(rg[i + 2 * j + 1]));
                  wu[j] = pack_bf16x2(__uint_as_float(ru[i + 2 * j]), __uint_as_float(ru[i + 2 * j + 1]));
                  const float2 g = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&wg[j]));
                  const float2 u = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&wu[j]));
                  // same rounding points as the standalone SwiGLU kernel: bit-identical results
                  const float sx = __bfloat162float(__float2bfloat16(g.x / (1.f + __expf(-g.x))));
                  const float sy = __bfloat162float(__float2bfloat16(g.y / (1.f + __expf(-g.y))));
                  wh[j] = pack_bf16x2(sx * u.x, sy * u.y);
                }
                if (staged) {
                  const int at = lane * 64 + (((i >> 3) ^ ((lane >> 1) & 3)) << 4);
                  *reinterpret_cast<uint4*>(slot + at) = pg;
                  *reinterpret_cast<uint4*>(slot + 2048 + at) = pu;
                  *reinterpret_cast<uint4*>(slot + 4096 + at) = ph;
                } else {
                  *reinterpret_cast<uint4*>(gu_row + col0 + i) = pg;
                  *reinterpret_cast<uint4*>(gu_row + p.gated_inter + col0 + i) = pu;
                  *reinterpret_cast<uint4*>(h_row + col0 + i) = ph;
                }
              }
              if (staged) {
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                  tma_store_2d(&p.map_out, slot, col0, band_row);
                  tma_store_2d(&p.map_up, slot + 2048, col0, band_row);
                  tma_store_2d(&p.map_h, slot + 4096, col0, band_row);
                  bulk_commit_group();
                }
                ++issued;
              }
            }
          } else {
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
              uint32_t r[32];
              tmem_ld_32x32(acc + c * 32, r);
              tmem_ld_wait();
              const int col0 = n0 + c * 32;
              if (staged ? (band_row >= p.M || col0 >= p.N) : (!row_ok || col0 >= p.N)) continue;
              float v[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
              if (p.bias != nullptr) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (col0 + i < p.N) v[i] += __ldg(p.bias + col0 + i);
              }
              if (staged) {
                // four 2 KB boxes per warp in rotation, one bulk group each
                uint8_t* slot = stage_base + (issued & 3) * 2048;
                if (lane == 0) bulk_wait_group_read<3>();
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                  uint4 pk;
                  pk.x = pack_bf16x2(v[i], v[i + 1]);
                  pk.y = pack_bf16x2(v[i + 2], v[i + 3]);
                  pk.z = pack_bf16x2(v[i + 4], v[i + 5]);
                  pk.w = pack_bf16x2(v[i + 6], v[i + 7]);
                  *reinterpret_cast<uint4*>(slot + lane * 64 +
                                            (((i >> 3) ^ ((lane >> 1) & 3)) << 4)) = pk;
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                  tma_store_2d(&p.map_out, slot, col0, band_row);
                  bulk_commit_group();
                }
                ++issued;
                continue;
              }
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + g_row * p.ldo + col0;
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                if (col0 + i >= p.N) break;
                uint4 pk;
                pk.x = pack_bf16x2(v[i], v[i + 1]);
                pk.y = pack_bf16x2(v[i + 2], v[i + 3]);
                pk.z = pack_bf16x2(v[i + 4], v[i + 5]);
                pk.w = pack_bf16x2(v[i + 6], v[i + 7]);
                *reinterpret_cast<uint4*>(o + i) = pk;
              }
            }
          }
        }
        tc_fence_before_sync();
        mbar_arrive(acc_empty);   // TMEM reads done (or skipped): the MMA warp may start the next round
        if (p.staged != 0) {
          // the stores must have read their boxes before any producer refills the weight stages
          if (lane == 0) bulk_wait_group_read<0>();
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      }
    }
    cp_async_wait<0>();
    if (lane == 0) bulk_wait_group<0>();   // staged stores written before the CTA retires
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int BN>
cudaError_t launch_bn(const AgGemmCall& c, int mt, int* status, cudaStream_t stream) {
  CUtensorMap ta;
  if (!make_bf16_tensor_map(&ta, c.a, c.M, c.K, c.lda, 64, kBM)) return cudaErrorInvalidValue;
  AgParams p{};
  p.w = c.w;
  p.out = c.out;
  p.bias = c.bias;
  p.gated_out = c.gated_out;
  p.ldo = c.ldo;
  p.gated_inter = c.gated_inter > 0 ? c.gated_inter : 0;
  p.M = c.M;
  p.N = c.N;
  p.K = c.K;
  p.mt = mt;
  p.status = status;
  p.map_out = p.map_up = p.map_h = ta;
  if (p.gated_inter > 0) {
    const __nv_bfloat16* gu = reinterpret_cast<const __nv_bfloat16*>(c.out);
    p.staged = make_bf16_store_map(&p.map_out, gu, c.M, p.gated_inter, c.ldo) &&
               make_bf16_store_map(&p.map_up, gu + p.gated_inter, c.M, p.gated_inter, c.ldo) &&
               make_bf16_store_map(&p.map_h, c.gated_out, c.M, p.gated_inter, p.gated_inter);
  } else {
    p.staged = make_bf16_store_map(&p.map_out, c.out, c.M, c.N, c.ldo);
  }
  auto kernel = gemm_allgather_kernel<BN>;
  constexpr int smem = AgSmem<BN>::kTotal;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  });
  if (attr_err != cudaSuccess) return attr_err;
  const int tile_cols = p.gated_inter > 0 ? BN / 2 : BN;
  const int span = p.gated_inter > 0 ? p.gated_inter : c.N;
  const int n_tiles = (span + tile_cols - 1) / tile_cols;
  const int grid = std::min(n_tiles, sm_count());
  kernel<<<grid, kThreads, smem, stream>>>(ta, p);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemm_allgather(const AgGemmCall& c, int* status, cudaStream_t stream) {
  auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
  if (c.M <= 0 || c.N <= 0 || c.K <= 0 || (c.K % 8) || (c.lda % 8) || (c.N % 8) || (c.ldo % 8) ||
      !aligned16(c.a) || !aligned16(c.out))
    return cudaErrorInvalidValue;
  const AgWeights& w = c.w;
  if (w.degree < 1 || w.degree > kMaxPeers || w.n_segs < 1 || w.n_segs > 4) return cudaErrorInvalidValue;
  const bool bf16_wire = w.shadow[0] != nullptr;
  int64_t rows = 0;
  for (int j = 0; j < w.n_segs; ++j) {
    const AgSegment& s = w.seg[j];
    if (s.rows <= 0 || s.q <= 0 || s.shard_off < 0 || s.full_off < 0 ||
        s.q * w.degree < static_cast<int64_t>(s.rows) * c.K ||
        static_cast<int64_t>(s.rows) * c.K >= (int64_t{1} << 31))   // 32-bit flat indices
      return cudaErrorInvalidValue;
    rows += s.rows;
  }
  if (rows != c.N) return cudaErrorInvalidValue;
  for (int r = 0; r < w.degree; ++r) {
    const void* base = bf16_wire ? static_cast<const void*>(w.shadow[r])
                                 : static_cast<const void*>(w.shard[r]);
    if (base == nullptr || !aligned16(base)) return cudaErrorInvalidValue;
  }
  if (w.full != nullptr && !aligned16(w.full)) return cudaErrorInvalidValue;
  const int m_tiles = (c.M + kBM - 1) / kBM;
  if (c.gated_inter > 0) {
    if (c.gated_out == nullptr || !aligned16(c.gated_out) || c.N != 2 * c.gated_inter ||
        (c.gated_inter % 8) || c.bias != nullptr || w.n_segs != 2 ||
        w.seg[0].rows != c.gated_inter || w.seg[1].rows != c.gated_inter)
      return cudaErrorInvalidValue;
    const int mt = std::min(m_tiles, 512 / 128);
    if (m_tiles > mt && w.full == nullptr) return cudaErrorInvalidValue;
    return launch_bn<128>(c, mt, status, stream);
  }
  // narrow tiles when the weight has few rows: more CTAs pulling, and up to eight row tiles of
  // A share one crossing of the link
  int bn = c.force_bn;
  if (bn == 0) bn = ((c.N + 127) / 128 >= sm_count() / 2 && m_tiles <= 4) ? 128 : 64;
  if (bn != 64 && bn != 128) return cudaErrorInvalidValue;
  const int mt = std::min(m_tiles, 512 / bn);
  if (m_tiles > mt && w.full == nullptr) return cudaErrorInvalidValue;
  return bn == 128 ? launch_bn<128>(c, mt, status, stream) : launch_bn<64>(c, mt, status, stream);
}

}  // namespace stb
