// bf16 x bf16 -> fp32 GEMM for sm_100a: TMA (local memory) -> 128-byte-swizzled shared memory ->
// tcgen05.mma with the accumulator in TMEM -> tcgen05.ld epilogue.
//
//   out[M,N] = sum_k A[m,k] * B[n,k]   (+ bias[n]) (+ residual[m,n]) (+ out[m,n] when accumulating)
//
// Either operand may be stored K-major ([rows, K], K contiguous) or MN-major ([K, rows], rows
// contiguous); the three combinations used by a linear layer's forward, dX and dW are
// (K,K), (K,MN) and (MN,MN).  This replaces the reference's F.linear / `@` call sites
// (src/sharded_runtime/runtime/qwen2_operators.py:55-64, 78-96, 122-125, 138-143).
//
// CTA = 6 warps: warp 0 issues TMA, warp 1 owns TMEM and issues MMAs (one lane), warps 2..5 are
// the epilogue (warp w reads TMEM lanes 32*(w%4)..+31, as the hardware requires).
#pragma once
#include "common.cuh"

namespace stb {

struct GemmEpilogue {
  void* out;              // bf16 or fp32, row-major [M, ldo]
  const float* bias;      // optional fp32 [N]
  const void* residual;   // optional, same dtype/ld as out
  const void* mul;        // unused by the plain epilogue (reserved for gated variants)
  int64_t ldo;            // leading dimension of out / residual (elements)
  int out_fp32;           // 1: fp32 output, 0: bf16 output
  int accumulate;         // 1: out += result (fp32 output only)
  float alpha;            // result scale applied before bias/residual
  // Sequence scatter (row-parallel GEMM -> reduce-scatter along the sequence): when
  // scatter_degree > 1 the fp32 result row m = b * scatter_seq + s goes to the buffer of the rank
  // that owns sequence position s, scatter_out[s / scatter_seq_local], at row
  // b * scatter_seq_local + s % scatter_seq_local.  The buffers may be peer memory: the partial
  // sums cross NVLink tile by tile from this epilogue, while later tiles are still in the MMAs.
  // Gated (SwiGLU) mode, gated_inter > 0: B is the fused [2 * inter, K] gate|up weight.  A tile
  // takes 128 gate rows and the 128 up rows of the same intermediate indices, so accumulator
  // columns 0..127 / 128..255 hold gate / up of one index range; the epilogue writes both halves
  // to `out` ([M, 2 * inter] bf16, gate|up as stored) and silu(gate) * up to `gated_out`
  // ([M, inter] bf16).
  void* gated_out;
  int gated_inter;
  float* scatter_out[8];
  int scatter_degree;
  int scatter_seq;
  int scatter_seq_local;
  // Broadcast variant (tensor parallelism without sequence parallelism: the partial sums are
  // all-reduced, every rank needs every row): row m is stored at row m of *every* scatter_out.
  int scatter_broadcast;
  // Staged store: the epilogue warps transpose each 32-row band through 128B-swizzled shared
  // memory and hand whole 32 x 128-byte boxes to TMA stores (`tma_c`), instead of every thread
  // storing 16-byte pieces of its own row.  Set by the launcher for plain bf16 / fp32 outputs
  // (no scatter, no gating, no accumulate) whose base and pitch TMA accepts.
  int staged_store;
};

// Tail split.  A persistent grid of G CTAs runs floor(tiles / G) full waves of whole tiles; the
// `tiles % G` tiles left over would occupy only part of the machine for a whole tile time, so
// each of them is cut along K into `split` units (rem * split <= G).  A split unit stores its raw
// fp32 accumulator tile in `workspace`; the unit that arrives last at the tile's counter adds the
// `split` partial tiles in index order (so the result does not depend on arrival order) and runs
// the normal epilogue.  Nothing waits on another CTA.
struct GemmSplit {
  int full_tiles;     // tiles [0, full_tiles) are whole-K units
  int split;          // K-splits per remaining tile (1: no tail split)
  int kb_per_split;   // k-blocks per split unit
  int total_units;
  float* workspace;   // [rem_tiles * split][128][BN] fp32
  int* counters;      // [rem_tiles], zero between launches
};

// Sequence all-gather fused into the GEMM that consumes the gathered activation (PULL variant).
// The A operand is the concatenation along the sequence of T ranks' [batch, seq_local, K] slices:
// row b * (T * seq_local) + r * seq_local + s of A is row b * seq_local + s of rank r's slice.
// Four extra warps of every CTA copy 8-row groups of A from the owners' buffers (plain 16-byte
// peer loads, twelve in flight per thread) into the local buffer `dst` that the A tensor map
// covers, and publish one flag per group; the TMA producer waits (bounded) for the flags of the
// rows a tile needs before it loads them.  Tiles whose rows have landed run while later groups
// are still crossing the link, so the transfer overlaps the MMAs tile by tile and the gathered
// activation stays in the local buffer for the GEMMs that reuse it.
//
// Flags hold the `epoch` of the launch that wrote them, so they never need clearing; every
// launch on a flag buffer must use a new epoch.  All CTAs of the grid must be able to become
// resident (the launcher keeps the grid at one CTA per SM) and two PULL GEMMs must not run
// concurrently on one device: a CTA waits for groups that other CTAs of its own grid pull.
struct GemmPull {
  const void* peers[8];   // rank r's [batch * seq_local, K] bf16 slice (row pitch `src_ld` elements)
  int degree;
  int batch;
  int seq_local;
  int64_t src_ld;         // elements
  void* dst;              // local [M, lda] bf16 buffer = the A operand
  int64_t dst_ld;
  uint32_t* flags;        // one per kPullRows-row group of A
  uint32_t epoch;
};
constexpr int kPullRows = 8;       // small groups: every CTA of the grid gets some to pull
constexpr int kPullThreads = 128;
constexpr int kPullBatch = 12;     // independent 16-byte loads per thread before the first store

constexpr int kGemmBM = 128;
constexpr int kGemmBK = 64;
constexpr int kGemmThreads = 192;

template <int BN>
struct GemmSmem {
  static constexpr int kABytes = kGemmBM * kGemmBK * 2;
  static constexpr int kBBytes = BN * kGemmBK * 2;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 192 ? 5 : 6);
  // TMEM allocations are powers of two: two 192-column accumulators live in a 512-column grant
  static constexpr int kTmemCols = (2 * BN <= 256) ? 256 : 512;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // tiles + barriers (full, empty, accumulator full/empty) + tmem pointer + abort flag, plus
  // 1 KB alignment slack
  // + 4 KB per epilogue warp to transpose scattered output rows into 128-byte row segments
  // (the staging area sits right after the operand tiles, so it is 1 KB aligned as the 128B
  // swizzle of the TMA stores needs; two buffers per warp where shared memory allows)
  static constexpr int kBarrierBytes = 256;
  static constexpr int kStoreBufs = (BN == 192) ? 1 : 2;
  static constexpr int kScatterStageBytes = 4 * kStoreBufs * 4096;
  static constexpr int kTotal = kStages * kStageBytes + 1024 + kBarrierBytes + kScatterStageBytes;
  static_assert(kTotal <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
};

template <int BN, bool A_MN, bool B_MN, bool PULL>
__device__ __forceinline__ void gemm_bf16_tcgen05_body(const CUtensorMap& tma_a,
                                                       const CUtensorMap& tma_b,
                                                       const CUtensorMap& tma_c,
                                                       const CUtensorMap& tma_c_up,
                                                       const CUtensorMap& tma_c_h,
                                                       const GemmEpilogue& ep, const GemmSplit& sp,
                                                       const GemmPull& pull, int M, int N, int K,
                                                       int* __restrict__ status) {
  // Persistent: each CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The accumulator is
  // double buffered in TMEM (2 x BN columns) so the epilogue of one tile overlaps the MMAs of the
  // next; the shared-memory operand pipeline runs across tile boundaries without draining.
  using S = GemmSmem<BN>;
  constexpr int STAGES = S::kStages;
  // an earlier kernel recorded a failure (a peer that never signalled, a wait that expired): the
  // operands may be stale, skip the work -- uniformly, before any barrier or TMEM exists
  if (kernel_should_skip(status)) return;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* tiles = smem;
  uint8_t* store_stage = smem + STAGES * S::kStageBytes;   // [4 warps][kStoreBufs][4 KB]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(store_stage + S::kScatterStageBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2], 128 arrivals each
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (M + kGemmBM - 1) / kGemmBM;
  const bool gated = ep.gated_inter > 0;
  const int tile_cols = gated ? BN / 2 : BN;          // output columns (per half) covered by a tile
  const int n_span = gated ? ep.gated_inter : N;
  const int n_tiles = (n_span + tile_cols - 1) / tile_cols;
  const int num_kb = (K + kGemmBK - 1) / kGemmBK;
  constexpr int GROUP = 8;
  const int group_span = GROUP * n_tiles;

  // Grouped rasterisation: walk up to 8 M-tiles before moving to the next N-tile so that the
  // CTAs resident at one time share operand tiles in L2.
  // unit -> (tile, k-block range, split index or -1 for a whole tile)
  auto unit_work = [&](int unit, int& tile, int& kb0, int& kb1, int& part) {
    if (unit < sp.full_tiles) {
      tile = unit; kb0 = 0; kb1 = num_kb; part = -1;
    } else {
      const int r = unit - sp.full_tiles;
      tile = sp.full_tiles + r / sp.split;
      part = sp.split > 1 ? r % sp.split : -1;
      kb0 = sp.split > 1 ? part * sp.kb_per_split : 0;
      kb1 = sp.split > 1 ? min(num_kb, kb0 + sp.kb_per_split) : num_kb;
    }
  };
  auto tile_origin = [&](int tile, int& m0, int& n0) {
    const int first_m = (tile / group_span) * GROUP;
    const int gm = min(m_tiles - first_m, GROUP);
    m0 = (first_m + (tile % group_span) % gm) * kGemmBM;
    n0 = ((tile % group_span) / gm) * tile_cols;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 128);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
    if (ep.staged_store) {
      prefetch_tensormap(&tma_c);
      if (ep.gated_inter > 0) {
        prefetch_tensormap(&tma_c_up);
        prefetch_tensormap(&tma_c_h);
      }
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, S::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;  // k-blocks issued so far, across tiles
      bool ok = true;
      uint64_t ready_tiles = 0;   // PULL: row tiles of A whose groups were all seen landed
      (void)ready_tiles;
      for (int unit = blockIdx.x; unit < sp.total_units && ok; unit += gridDim.x) {
        int tile, kb0, kb1, part, m0, n0;
        unit_work(unit, tile, kb0, kb1, part);
        tile_origin(tile, m0, n0);
        if constexpr (PULL) {
          // The rows m0 .. m0 + 127 of A must have landed in the local buffer.  All flags of the
          // tile are read in one batch of independent relaxed loads (an acquire load per flag
          // would serialise sixteen L2 round trips); one fence then orders the tile's TMA reads
          // behind them.  Row tiles already seen complete are remembered.
          const int m_tile = m0 / kGemmBM;
          const bool known = m_tile < 64 && ((ready_tiles >> m_tile) & 1ull);
          if (!known) {
            const int g_first = m0 / kPullRows;
            const int g_count = (min(M, m0 + kGemmBM) - 1) / kPullRows - g_first + 1;
            const uint64_t t0 = global_ns();
            for (uint32_t spin = 0;; ++spin) {
              uint32_t seen[kGemmBM / kPullRows];
#pragma unroll
              for (int g = 0; g < kGemmBM / kPullRows; ++g) {
                seen[g] = pull.epoch;
                if (g < g_count)
                  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];"
                               : "=r"(seen[g]) : "l"(pull.flags + g_first + g) : "memory");
              }
              bool all = true;
#pragma unroll
              for (int g = 0; g < kGemmBM / kPullRows; ++g) all = all && seen[g] == pull.epoch;
              if (all) break;
              if ((spin & 63u) == 63u &&
                  (status_failed(status) || global_ns() - t0 > kWaitBudgetNs)) {
                if (status != nullptr) atomicCAS(status, kOk, kErrPullWait);
                *abort_flag = 1;
                ok = false;
                break;
              }
              __nanosleep(32);
            }
            if (!ok) break;
            if (m_tile < 64) ready_tiles |= 1ull << m_tile;
            asm volatile("fence.acq_rel.gpu;" ::: "memory");
            // generic-proxy stores of the pulling warps -> visible to the TMA (async proxy) reads
            asm volatile("fence.proxy.async;" ::: "memory");
          }
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, status, kErrProducerEmptyWait)) {
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = tiles + s * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          mbar_expect_tx(&full_bar[s], S::kStageBytes);
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tma_a, &full_bar[s], kb * kGemmBK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < kGemmBM / 64; ++c)
              tma_load_2d(sa + c * 8192, &tma_a, &full_bar[s], m0 + c * 64, kb * kGemmBK);
          }
          if constexpr (!B_MN) {
            if (gated) {   // box of BN / 2 rows: gate rows, then the matching up rows
              tma_load_2d(sb, &tma_b, &full_bar[s], kb * kGemmBK, n0);
              tma_load_2d(sb + (BN / 2) * 128, &tma_b, &full_bar[s], kb * kGemmBK,
                          ep.gated_inter + n0);
            } else {
              tma_load_2d(sb, &tma_b, &full_bar[s], kb * kGemmBK, n0);
            }
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * 8192, &tma_b, &full_bar[s], n0 + c * 64, kb * kGemmBK);
          }
        }
      }
      // Error path only: wait (bounded) for copies this thread issued that nobody consumed.
      if (*abort_flag) {
        for (int k = max(0, it - STAGES); k < it; ++k)
          mbar_wait(&full_bar[k % STAGES], (k / STAGES) & 1, status, kErrDrainWait);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kGemmBM, BN, A_MN, B_MN);
      int it = 0, local = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < sp.total_units && ok; unit += gridDim.x, ++local) {
        int tile, kb0, kb1, part;
        unit_work(unit, tile, kb0, kb1, part);
        const int ab = local & 1;
        // the epilogue must have drained this accumulator buffer (two tiles ago)
        if (!mbar_wait(&acc_empty[ab], ((local >> 1) & 1) ^ 1, status, kErrMmaFullWait)) {
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + ab * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, status, kErrMmaFullWait)) {
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(tiles + s * S::kStageBytes);
          const uint32_t b_base = a_base + S::kABytes;
#pragma unroll
          for (int k = 0; k < kGemmBK / 16; ++k) {
            // K-major: the 16-element K slice is 32 bytes further along each 128-byte row.
            // MN-major: the slice is 16 K-rows (two 8-row swizzle atoms, 1024 B apart) further
            // on; 64-wide MN chunks sit 8192 B apart (the leading-dimension byte offset).
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_base + k * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_base + k * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(b_base + k * 32, 16, 1024);
            tc_mma_f16(tmem_d, da, db, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
        }
        tc_commit(&acc_full[ab]);
      }
    }
  } else if (PULL && warp >= 6) {
    // Pull warps: copy groups of rows of A from their owners into the local buffer, lowest groups
    // first (the order in which the tiles of the first wave need them), then publish the flag.
    const int t = threadIdx.x - kGemmThreads;              // 0..127
    const int seq = pull.degree * pull.seq_local;
    const int chunks_per_row = (K * 2) / 16;               // 16-byte pieces of a row (K % 8 == 0)
    const int groups = (M + kPullRows - 1) / kPullRows;
    for (int g = blockIdx.x; g < groups; g += gridDim.x) {
      const int row0 = g * kPullRows;
      const int rows = min(kPullRows, M - row0);
      const int total = rows * chunks_per_row;
      for (int i0 = t; i0 < total; i0 += kPullThreads * kPullBatch) {
        uint4 v[kPullBatch];
#pragma unroll
        for (int u = 0; u < kPullBatch; ++u) {
          const int i = i0 + u * kPullThreads;
          if (i < total) {
            const int r = row0 + i / chunks_per_row, c = i % chunks_per_row;
            const int b = r / seq, pos = r - b * seq;
            const int owner = pos / pull.seq_local;
            const int64_t src_row = static_cast<int64_t>(b) * pull.seq_local + (pos - owner * pull.seq_local);
            v[u] = *(reinterpret_cast<const uint4*>(
                         reinterpret_cast<const __nv_bfloat16*>(pull.peers[owner]) +
                         src_row * pull.src_ld) + c);
          }
        }
#pragma unroll
        for (int u = 0; u < kPullBatch; ++u) {
          const int i = i0 + u * kPullThreads;
          if (i < total) {
            const int r = row0 + i / chunks_per_row, c = i % chunks_per_row;
            *(reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(pull.dst) +
                                       static_cast<int64_t>(r) * pull.dst_ld) + c) = v[u];
          }
        }
      }
      __threadfence();                                      // the group's rows before its flag
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (t == 0)
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(pull.flags + g), "r"(pull.epoch)
                     : "memory");
    }
  } else {
    // Epilogue: 4 warps x 32 lanes = the 128 accumulator rows.
    const int q = warp & 3;
    const int row = q * 32 + lane;
    int local = 0;
    int sbuf = 0;          // staged store: which of this warp's staging buffers is written next
    bool ok = true;
    int* last_flag = reinterpret_cast<int*>(tmem_ptr + 2);   // shared: "this CTA reduces the tile"
    for (int unit = blockIdx.x; unit < sp.total_units; unit += gridDim.x, ++local) {
      int tile, kb0, kb1, part, m0, n0;
      unit_work(unit, tile, kb0, kb1, part);
      tile_origin(tile, m0, n0);
      const int ab = local & 1;
      if (ok) ok = mbar_wait(&acc_full[ab], (local >> 1) & 1, status, kErrEpilogueAccumWait);
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + ab * BN;
      const int64_t g_row = static_cast<int64_t>(m0) + row;
      const bool row_ok = ok && g_row < M;
      const bool warp_ok = __all_sync(0xffffffffu, ok);
      // Scatter epilogue: after the shared-memory transpose lane l stores rows 4k + l/8 (k = 0..7)
      // of its warp's 32-row band; their destinations (owner buffer, row inside it) do not
      // depend on the column chunk, so they are resolved once per tile.
      float* scatter_row[8];
      if (ep.scatter_degree > 1) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int gr = m0 + q * 32 + k * 4 + (lane >> 3);
          scatter_row[k] = nullptr;
          if (ok && gr < M) {
            if (ep.scatter_broadcast) {
              // the row inside destination 0; the other destinations use the same offset
              scatter_row[k] = ep.scatter_out[0] + static_cast<int64_t>(gr) * ep.ldo;
            } else {
              const int b = gr / ep.scatter_seq;
              const int pos = gr - b * ep.scatter_seq;
              const int owner = pos / ep.scatter_seq_local;
              scatter_row[k] = ep.scatter_out[owner] +
                               (static_cast<int64_t>(b) * ep.scatter_seq_local +
                                (pos - owner * ep.scatter_seq_local)) * ep.ldo;
            }
          }
        }
      }
      // one 32-column chunk of this thread's accumulator row -> output (all epilogue variants)
      auto emit = [&](uint32_t (&r)[32], int c) {
        const int col0 = n0 + c * 32;
        if (col0 >= N) return;                         // warp-uniform
        if (ep.scatter_degree > 1) {
          // Sequence scatter.  A thread owns one accumulator row, so storing from registers
          // would emit 16-byte pieces of 32 different rows per instruction -- fine for local
          // L2, ruinous for stores that cross NVLink.  The warp's 32x32 block goes through
          // shared memory (XOR-swizzled 16-byte slots, conflict free both ways) and leaves as
          // four full 128-byte row segments per instruction.
          float* stage = reinterpret_cast<float*>(store_stage) + q * (S::kStoreBufs * 1024);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 x;
            x.x = __uint_as_float(r[4 * j]) * ep.alpha;
            x.y = __uint_as_float(r[4 * j + 1]) * ep.alpha;
            x.z = __uint_as_float(r[4 * j + 2]) * ep.alpha;
            x.w = __uint_as_float(r[4 * j + 3]) * ep.alpha;
            *reinterpret_cast<float4*>(stage + lane * 32 + ((j ^ (lane & 7)) << 2)) = x;
          }
          __syncwarp();
          const int seg = lane & 7;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int rr = k * 4 + (lane >> 3);
            const float4 x =
                *reinterpret_cast<const float4*>(stage + rr * 32 + ((seg ^ (rr & 7)) << 2));
            if (scatter_row[k] != nullptr && col0 + seg * 4 < N) {
              if (ep.scatter_broadcast) {
                const int64_t off = (scatter_row[k] - ep.scatter_out[0]) + col0 + seg * 4;
                for (int o = 0; o < ep.scatter_degree; ++o)
                  *reinterpret_cast<float4*>(ep.scatter_out[o] + off) = x;
              } else {
                *reinterpret_cast<float4*>(scatter_row[k] + col0 + seg * 4) = x;
              }
            }
          }
          __syncwarp();
          return;
        }
        if (ep.staged_store) {
          // Staged store.  Rows past M and columns past N may hold anything in shared memory:
          // the TMA store does not write the part of a box that lies outside the tensor.
          const int band_row = m0 + q * 32;
          if (!warp_ok || band_row >= M) return;          // warp-uniform
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * ep.alpha;
          if (ep.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < N) v[i] += __ldg(ep.bias + col0 + i);
          }
          uint8_t* stage = store_stage + (q * S::kStoreBufs + sbuf) * 4096;
          if (ep.out_fp32) {
            if (ep.residual != nullptr && row_ok) {
              const float* rs = reinterpret_cast<const float*>(ep.residual) + g_row * ep.ldo + col0;
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                if (col0 + i >= N) break;
                const float4 y = *reinterpret_cast<const float4*>(rs + i);
                v[i] += y.x; v[i + 1] += y.y; v[i + 2] += y.z; v[i + 3] += y.w;
              }
            }
            // the store that last read this buffer must have finished reading it
            if (lane == 0) bulk_wait_group_read<S::kStoreBufs - 1>();
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<float4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                  make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tma_c, stage, col0, band_row);
              bulk_commit_group();
            }
            sbuf = (sbuf + 1) % S::kStoreBufs;
            return;
          }
          // bf16: two 32-column chunks fill the two halves of one buffer of 128-byte rows
          if (ep.residual != nullptr && row_ok) {
            const __nv_bfloat16* rs =
                reinterpret_cast<const __nv_bfloat16*>(ep.residual) + g_row * ep.ldo + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (col0 + i >= N) break;
              const uint4 y = *reinterpret_cast<const uint4*>(rs + i);
              const __nv_bfloat162* yb = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(yb[j]);
                v[i + 2 * j] += f.x;
                v[i + 2 * j + 1] += f.y;
              }
            }
          }
          const int half = c & 1;
          if (half == 0) {
            if (lane == 0) bulk_wait_group_read<S::kStoreBufs - 1>();
            __syncwarp();
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 pk;
            pk.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
            pk.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
            pk.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
            pk.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
            *reinterpret_cast<uint4*>(stage + lane * 128 + (((half * 4 + j) ^ (lane & 7)) << 4)) = pk;
          }
          if (half == 1 || col0 + 32 >= N) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tma_c, stage, col0 - half * 32, band_row);
              bulk_commit_group();
            }
            sbuf = (sbuf + 1) % S::kStoreBufs;
          }
          return;
        }
        if (!row_ok) return;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * ep.alpha;
        if (ep.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + i < N) v[i] += __ldg(ep.bias + col0 + i);
        }
        if (ep.out_fp32) {
          float* o = reinterpret_cast<float*>(ep.out) + g_row * ep.ldo + col0;
          const float* rs = ep.residual ? reinterpret_cast<const float*>(ep.residual) +
                                              g_row * ep.ldo + col0
                                        : nullptr;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            if (col0 + i >= N) break;
            float4 x = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            if (rs) {
              const float4 y = *reinterpret_cast<const float4*>(rs + i);
              x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
            }
            if (ep.accumulate) {
              const float4 y = *reinterpret_cast<const float4*>(o + i);
              x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
            }
            *reinterpret_cast<float4*>(o + i) = x;
          }
        } else {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(ep.out) + g_row * ep.ldo + col0;
          const __nv_bfloat16* rs =
              ep.residual
                  ? reinterpret_cast<const __nv_bfloat16*>(ep.residual) + g_row * ep.ldo + col0
                  : nullptr;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            if (col0 + i >= N) break;
            if (rs) {
              const uint4 y = *reinterpret_cast<const uint4*>(rs + i);
              const __nv_bfloat162* yb = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(yb[j]);
                v[i + 2 * j] += f.x;
                v[i + 2 * j + 1] += f.y;
              }
            }
            uint4 pk;
            pk.x = pack_bf16x2(v[i], v[i + 1]);
            pk.y = pack_bf16x2(v[i + 2], v[i + 3]);
            pk.z = pack_bf16x2(v[i + 4], v[i + 5]);
            pk.w = pack_bf16x2(v[i + 6], v[i + 7]);
            *reinterpret_cast<uint4*>(o + i) = pk;
          }
        }
      };
      if (gated) {
        // SwiGLU epilogue: columns c*32.. of the gate half pair with the same columns of the up
        // half.  Both are rounded to bf16 first (that is what the backward reads back), then
        // h = bf16(silu(gate)) * up is rounded once more.
        __nv_bfloat16* gu_row = reinterpret_cast<__nv_bfloat16*>(ep.out) + g_row * ep.ldo;
        __nv_bfloat16* h_row =
            reinterpret_cast<__nv_bfloat16*>(ep.gated_out) + g_row * ep.gated_inter;
        const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(tmem_d + lane_base + c * 32, rg);
          tmem_ld_32x32(tmem_d + lane_base + BN / 2 + c * 32, ru);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          const bool staged = ep.staged_store != 0;        // warp-uniform
          if (staged ? (!warp_ok || m0 + q * 32 >= M || col0 >= ep.gated_inter)
                     : (!row_ok || col0 >= ep.gated_inter))
            continue;
          // Staged: three 32 x 64-byte boxes (gate, up, product) in 64B-swizzled shared memory,
          // one bulk group per chunk; the previous chunk's boxes were read while this chunk's
          // values were computed above.
          uint8_t* slot = store_stage + q * (S::kStoreBufs * 4096);
          if (staged) {
            if (lane == 0) bulk_wait_group_read<0>();
            __syncwarp();
          }
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            if (!staged && col0 + i >= ep.gated_inter) break;
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
              // silu(gate) is rounded to bf16 before the product, as under bf16 autocast
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
              *reinterpret_cast<uint4*>(gu_row + ep.gated_inter + col0 + i) = pu;
              *reinterpret_cast<uint4*>(h_row + col0 + i) = ph;
            }
          }
          if (staged) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              const int band_row = m0 + q * 32;
              tma_store_2d(&tma_c, slot, col0, band_row);
              tma_store_2d(&tma_c_up, slot + 2048, col0, band_row);
              tma_store_2d(&tma_c_h, slot + 4096, col0, band_row);
              bulk_commit_group();
            }
          }
        }
        tc_fence_before_sync();
        mbar_arrive(&acc_empty[ab]);
        continue;
      }
      if (part < 0) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_d + (static_cast<uint32_t>(q * 32) << 16) + c * 32, r);
          tmem_ld_wait();
          emit(r, c);
        }
        tc_fence_before_sync();
        mbar_arrive(&acc_empty[ab]);   // TMEM reads complete: hand the buffer back to the MMA warp
        continue;
      }
      // ---- K-split unit: park the raw partial tile, the last arrival reduces
      // Workspace layout per partial tile: [BN / 4 column quads][128 rows][4 floats], so the 32
      // lanes of a warp (consecutive rows) touch consecutive 16-byte words both when parking
      // and when reducing; the thread that reduces a row is the one that owns it in every unit.
      const int rem_tile = tile - sp.full_tiles;
      constexpr int64_t kTileFloats = static_cast<int64_t>(kGemmBM) * BN;
      float* mine = sp.workspace + (static_cast<int64_t>(rem_tile) * sp.split + part) * kTileFloats +
                    row * 4;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_d + (static_cast<uint32_t>(q * 32) << 16) + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(mine + (c * 8 + j) * (kGemmBM * 4)) =
              make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
      }
      tc_fence_before_sync();
      mbar_arrive(&acc_empty[ab]);
      __threadfence();                              // partial tile visible before the count
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        const int seen = atomicAdd(sp.counters + rem_tile, 1);
        *last_flag = (seen == sp.split - 1) ? 1 : 0;
        if (seen == sp.split - 1) sp.counters[rem_tile] = 0;   // ready for the next launch
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*last_flag == 0) continue;
      __threadfence();
      const float* first = sp.workspace + static_cast<int64_t>(rem_tile) * sp.split * kTileFloats +
                           row * 4;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        float acc[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = 0.f;
        for (int sidx = 0; sidx < sp.split; ++sidx) {
          const float* src = first + sidx * kTileFloats;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 t = __ldcg(reinterpret_cast<const float4*>(src + (c * 8 + j) * (kGemmBM * 4)));
            acc[4 * j] += t.x; acc[4 * j + 1] += t.y; acc[4 * j + 2] += t.z; acc[4 * j + 3] += t.w;
          }
        }
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(acc[i]);
        emit(r, c);
      }
    }
    // this warp's staged stores must have read their shared memory and written their rows
    // before the CTA retires
    if (lane == 0) bulk_wait_group<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, S::kTmemCols);
  }
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a,
                         const __grid_constant__ CUtensorMap tma_b,
                         const __grid_constant__ CUtensorMap tma_c,
                         const __grid_constant__ CUtensorMap tma_c_up,
                         const __grid_constant__ CUtensorMap tma_c_h, GemmEpilogue ep, GemmSplit sp,
                         int M, int N, int K, int* __restrict__ status) {
  gemm_bf16_tcgen05_body<BN, A_MN, B_MN, false>(tma_a, tma_b, tma_c, tma_c_up, tma_c_h, ep, sp,
                                                GemmPull{}, M, N, K, status);
}

// The same GEMM with four more warps that pull the A operand from its owners (see GemmPull).
template <int BN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads + kPullThreads, 1)
gemm_pull_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a,
                              const __grid_constant__ CUtensorMap tma_b,
                              const __grid_constant__ CUtensorMap tma_c,
                              const __grid_constant__ CUtensorMap tma_c_up,
                              const __grid_constant__ CUtensorMap tma_c_h, GemmEpilogue ep,
                              GemmSplit sp, GemmPull pull, int M, int N, int K,
                              int* __restrict__ status) {
  gemm_bf16_tcgen05_body<BN, false, B_MN, true>(tma_a, tma_b, tma_c, tma_c_up, tma_c_h, ep, sp, pull,
                                                M, N, K, status);
}

}  // namespace stb
