// Causal grouped-query attention for head_dim 128 on sm_100a: forward, and backward as two
// kernels (dK/dV per key block, dQ per query block).  All five/seven matrix products run on
// tcgen05 with accumulators in TMEM; Q/K/V/dO tiles arrive by TMA from the packed, rope-applied
// qkv buffer; the softmax warps read scores from TMEM with tcgen05.ld and hand P / dS back to the
// tensor core through 128-byte-swizzled shared memory.  No S x S matrix ever reaches global
// memory (the reference materialises it: src/sharded_runtime/models/qwen2.py:247-257).
//
// Tile = 128 x 128 (rows x head_dim or rows x rows) bf16, held as two 64-column halves of 16 KB
// (128 rows x 128 bytes, TMA SWIZZLE_128B).  The same tile serves as a K-major operand (reduction
// over its columns) or an MN-major operand (reduction over its rows); only the descriptor differs.
//
// CTA = 6 warps: 0 = TMA producer, 1 = MMA issuer / TMEM owner, 2..5 = softmax (one row each).
// Every mbarrier wait is bounded; on expiry the status word is set and the roles fall through.
#include "api.h"
#include "common.cuh"

namespace stb {

bool make_bf16_tensor_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols,
                          int64_t ld, int box_cols, int box_rows);

namespace {

constexpr int kD = 128;          // head dim
constexpr int kBlk = 128;        // rows per tile
constexpr int kHalf = 16384;     // bytes of one 64-column half tile
constexpr int kTile = 2 * kHalf;
constexpr int kThreads = 192;

// k-th 16-wide reduction slice of a tile used K-major (reduce over columns).
__device__ __forceinline__ uint64_t desc_k(uint32_t tile, int kk) {
  return make_smem_desc_sw128(tile + (kk >> 2) * kHalf + (kk & 3) * 32, 16, 1024);
}
// k-th 16-row reduction slice of a tile used MN-major (reduce over rows).
__device__ __forceinline__ uint64_t desc_mn(uint32_t tile, int kk) {
  return make_smem_desc_sw128(tile + kk * 2048, kHalf, 1024);
}

// D[128x128] (+)= A * B over a 128-long reduction: 8 MMAs of K = 16.
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void mma_128(uint32_t tmem_d, uint32_t a_tile, uint32_t b_tile,
                                        bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(128, 128, A_MN, B_MN);
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint64_t da = A_MN ? desc_mn(a_tile, kk) : desc_k(a_tile, kk);
    const uint64_t db = B_MN ? desc_mn(b_tile, kk) : desc_k(b_tile, kk);
    tc_mma_f16(tmem_d, da, db, idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}

// TMA: one 128x128 tile = two boxes of 64 columns.
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar,
                                          int col, int row) {
  tma_load_2d(dst, map, bar, col, row);
  tma_load_2d(dst + kHalf, map, bar, col + 64, row);
}

// Store 8 bf16 values (columns c8*8 .. +7 of row r) into a swizzled K-major tile.
__device__ __forceinline__ void store_row8(uint8_t* tile, int r, int c8, uint4 v) {
  const int half = c8 >> 3, chunk = c8 & 7;
  *reinterpret_cast<uint4*>(tile + half * kHalf + r * 128 + ((chunk ^ (r & 7)) << 4)) = v;
}

__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct FwdParams {
  __nv_bfloat16* out;
  float* lse;
  const uint8_t* key_mask;
  int batch, seq, hq, hkv;
  float scale;
  int* status;
  const uint32_t* key_bits;   // packed key mask (bit i of word w = key 32 w + i), see pack_key_mask
  int bits_pitch;             // words per sample, a multiple of 4
};

// The 128 mask bits of key block j of sample b; all ones without a mask.  With a byte mask the
// bits are assembled on the fly (slow path kept for callers that did not pack the mask).
__device__ __forceinline__ void load_key_bits(const uint32_t* bits, int pitch, const uint8_t* bytes,
                                              int seq, int b, int j, uint32_t (&w)[4]) {
  if (bits != nullptr) {
    const uint4 v = *reinterpret_cast<const uint4*>(bits + static_cast<int64_t>(b) * pitch + j * 4);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  } else if (bytes != nullptr) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t word = 0;
      for (int i = 0; i < 32; ++i) {
        const int kv = j * 128 + c * 32 + i;
        word |= (kv < seq && bytes[static_cast<int64_t>(b) * seq + kv] != 0) ? (1u << i) : 0u;
      }
      w[c] = word;
    }
  } else {
    w[0] = w[1] = w[2] = w[3] = 0xffffffffu;
  }
}

// smem: Q tile | K,V x 2 stages | P tile | barriers
constexpr int kFwdSmem = kTile + 4 * kTile + kTile + 1024 + 256;

__global__ void __launch_bounds__(kThreads, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap map, FwdParams p) {
  if (kernel_should_skip(p.status)) return;   // an earlier kernel already failed
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + kTile;          // stage s: K at sKV + s*2*kTile, V right after
  uint8_t* sP = sKV + 4 * kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kTile);
  uint64_t* q_full = bars;            // 1
  uint64_t* kv_full = bars + 1;       // 2
  uint64_t* kv_empty = bars + 3;      // 2
  uint64_t* s_full = bars + 5;        // 2: scores are double buffered in TMEM
  uint64_t* p_full = bars + 7;        // 1 (128 arrivals)
  uint64_t* o_done = bars + 8;        // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.hq / p.hkv);
  const int n_kv = qb + 1;  // causal: key blocks 0..qb
  const int row0 = b * p.seq;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(p_full, 128);
    mbar_init(o_done, 1);
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&map);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // S(j) lives in columns (j & 1) * 128: Q K^T of key block j + 1 is issued before the softmax of
  // block j has finished, so the tensor pipe works under the softmax instead of after it
  const uint32_t tS0 = tmem, tO = tmem + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, kTile);
      load_tile(sQ, &map, q_full, h * kD, row0 + qb * kBlk);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, p.status, kErrAttnWait)) break;
        uint8_t* k_dst = sKV + s * 2 * kTile;
        mbar_expect_tx(&kv_full[s], 2 * kTile);
        load_tile(k_dst, &map, &kv_full[s], (p.hq + hk) * kD, row0 + j * kBlk);
        load_tile(k_dst + kTile, &map, &kv_full[s], (p.hq + p.hkv + hk) * kD, row0 + j * kBlk);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, p.status, kErrAttnWait);
      if (ok) ok = mbar_wait(&kv_full[0], 0, p.status, kErrAttnWait);
      if (ok) {
        tc_fence_after_sync();
        mma_128<false, false>(tS0, smem_u32(sQ), smem_u32(sKV), false);          // S(0) = Q K_0^T
        tc_commit(&s_full[0]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        const uint32_t k_tile = smem_u32(sKV + s * 2 * kTile);
        if (j + 1 < n_kv) {
          // S(j+1) into the other score buffer: its last reader, the softmax of block j-1,
          // finished before p_full(j-1), which this thread has already waited for
          const int s1 = (j + 1) & 1;
          ok = mbar_wait(&kv_full[s1], ((j + 1) >> 1) & 1, p.status, kErrAttnWait);
          if (!ok) break;
          tc_fence_after_sync();
          mma_128<false, false>(tS0 + s1 * 128, smem_u32(sQ), smem_u32(sKV + s1 * 2 * kTile), false);
          tc_commit(&s_full[s1]);
        }
        ok = mbar_wait(p_full, j & 1, p.status, kErrAttnWait);       // P in smem, O rescaled
        if (!ok) break;
        tc_fence_after_sync();
        mma_128<false, true>(tO, smem_u32(sP), k_tile + kTile, j > 0);  // O += P V
        tc_commit(&kv_empty[s]);
        tc_commit(o_done);
      }
      if (!ok) {  // let the softmax warps fall through their bounded waits quickly
        tc_commit(&s_full[0]);
        tc_commit(&s_full[1]);
        tc_commit(o_done);
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;                 // row inside the tile
    const int q_idx = qb * kBlk + r;             // position inside the sequence
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, p.status, kErrAttnWait);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t tS = tS0 + (j & 1) * 128;
      const bool diag = (j == qb);
      // the whole score row (128 fp32) is read from TMEM once and kept in registers: four loads in
      // flight, one wait, no second pass over TMEM for the exponentials
      uint32_t sv[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(tS + lane_base + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[c * 32]));
      tmem_ld_wait();
      // the block's 128 key-mask bits: one 16-byte load per thread (same address for the whole
      // warp), and a block with every key visible takes the mask-free path
      uint32_t mw[4];
      load_key_bits(p.key_bits, p.bits_pitch, p.key_mask, p.seq, b, j, mw);
      const bool all_on = (mw[0] & mw[1] & mw[2] & mw[3]) == 0xffffffffu;
      const bool plain = !diag && all_on;     // every key of the block is visible
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 128; ++i) {
        const int kv = j * kBlk + i;
        const bool keep = plain || ((!diag || kv <= q_idx) && ((mw[i >> 5] >> (i & 31)) & 1u));
        const float x = keep ? __uint_as_float(sv[i]) * p.scale : -INFINITY;
        sv[i] = __float_as_uint(x);
        mx = fmaxf(mx, x);
      }
      const float m_new = fmaxf(m, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m == -INFINITY) ? 0.f : __expf(m - m_use);
      // probabilities, rounded to bf16 and packed (masked scores are -inf: exp gives 0); kept in
      // registers until the previous P V has released the shared-memory P tile
      float sum = 0.f;
      uint32_t pk[64];
#pragma unroll
      for (int i = 0; i < 128; i += 2) {
        const float x0 = __uint_as_float(sv[i]), x1 = __uint_as_float(sv[i + 1]);
        float e0 = (x0 == -INFINITY) ? 0.f : __expf(x0 - m_use);
        float e1 = (x1 == -INFINITY) ? 0.f : __expf(x1 - m_use);
        // sum what the tensor core will see (bf16-rounded), as the normaliser
        e0 = __bfloat162float(__float2bfloat16(e0));
        e1 = __bfloat162float(__float2bfloat16(e1));
        sum += e0 + e1;
        pk[i >> 1] = pack_bf16x2(e0, e1);
      }
      if (j > 0) {
        // previous P V finished (o_done), so O may be rescaled in place and P overwritten; the
        // score registers are dead by now, so the whole O row (128 fp32) fits in registers
        ok = mbar_wait(o_done, (j - 1) & 1, p.status, kErrAttnWait);
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
          uint32_t ov[128];
#pragma unroll
          for (int c = 0; c < 4; ++c)
            tmem_ld_32x32(tO + lane_base + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&ov[c * 32]));
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 128; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
#pragma unroll
          for (int c = 0; c < 4; ++c)
            tmem_st_32x32(tO + lane_base + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&ov[c * 32]));
          tmem_st_wait();
        }
      }
#pragma unroll
      for (int g = 0; g < 16; ++g)
        store_row8(sP, r, g, make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]));
      l = l * alpha + sum;
      m = m_new;
      tc_fence_before_sync();
      fence_proxy_async();   // generic-proxy writes of P must be visible to the MMA's async proxy
      mbar_arrive(p_full);
    }
    // epilogue: O / l -> bf16
    if (ok) ok = mbar_wait(o_done, (n_kv - 1) & 1, p.status, kErrAttnWait);
    tc_fence_after_sync();
    const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
    const bool store = ok && q_idx < p.seq;
    __nv_bfloat16* orow = p.out + (static_cast<int64_t>(row0 + q_idx) * p.hq + h) * kD;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t v[32];
      tmem_ld_32x32(tO + lane_base + c * 32, v);
      tmem_ld_wait();
      if (store) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 pk;
          pk.x = pack_bf16x2(__uint_as_float(v[8 * g]) * inv_l, __uint_as_float(v[8 * g + 1]) * inv_l);
          pk.y = pack_bf16x2(__uint_as_float(v[8 * g + 2]) * inv_l, __uint_as_float(v[8 * g + 3]) * inv_l);
          pk.z = pack_bf16x2(__uint_as_float(v[8 * g + 4]) * inv_l, __uint_as_float(v[8 * g + 5]) * inv_l);
          pk.w = pack_bf16x2(__uint_as_float(v[8 * g + 6]) * inv_l, __uint_as_float(v[8 * g + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = pk;
        }
      }
    }
    if (store)
      p.lse[(static_cast<int64_t>(b) * p.hq + h) * p.seq + q_idx] = (l > 0.f) ? m + __logf(l) : 0.f;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]   (one warp per (row, head))
__global__ void attention_delta_kernel(const __nv_bfloat16* __restrict__ out,
                                       const __nv_bfloat16* __restrict__ dout,
                                       float* __restrict__ delta, int batch, int seq, int hq) {
  const int64_t w = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t total = static_cast<int64_t>(batch) * seq * hq;
  if (w >= total) return;
  const int64_t row = w / hq;
  const int h = static_cast<int>(w % hq);
  const uint2 a = *reinterpret_cast<const uint2*>(out + w * kD + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(dout + w * kD + lane * 4);
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g.x));
  const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g.y));
  float s = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) {
    const int64_t b = row / seq, sidx = row % seq;
    delta[(b * hq + h) * seq + sidx] = s;
  }
}

struct BwdParams {
  const float* lse;
  const float* delta;
  __nv_bfloat16* dqkv;
  const uint8_t* key_mask;
  int batch, seq, hq, hkv;
  float scale;
  int* status;
  float* dkv_part;   // [parts, batch*seq, 2*hkv*128] fp32 partial dK|dV when the group is split
  int parts;         // CTAs sharing one kv head's query-head group (1: write bf16 directly)
  const uint32_t* key_bits;
  int bits_pitch;
};

// ---------------------------------------------------------------------------- dQ
// One CTA per (query block, query head, batch).  Per key block j <= i:
//   S = Q K^T, dP = dO V^T  ->  dS = P * (dP - delta) * scale  ->  dQ += dS K.
// smem: Q | dO | K | V | dS | barriers
constexpr int kDqSmem = 5 * kTile + 1024 + 256;

__global__ void __launch_bounds__(kThreads, 1)
attention_dq_kernel(const __grid_constant__ CUtensorMap map_qkv,
                    const __grid_constant__ CUtensorMap map_do, BwdParams p) {
  if (kernel_should_skip(p.status)) return;   // an earlier kernel already failed
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + kTile;
  uint8_t* sK = sdO + kTile;
  uint8_t* sV = sK + kTile;
  uint8_t* sdS = sV + kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + kTile);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* ds_full = bars + 4;   // 128 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.hq / p.hkv);
  const int n_kv = qb + 1;
  const int row0 = b * p.seq;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(kv_full, 1);
    mbar_init(kv_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(ds_full, 128);
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 128, tdQ = tmem + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * kTile);
      load_tile(sQ, &map_qkv, q_full, h * kD, row0 + qb * kBlk);
      load_tile(sdO, &map_do, q_full, h * kD, row0 + qb * kBlk);
      for (int j = 0; j < n_kv; ++j) {
        if (!mbar_wait(kv_empty, (j & 1) ^ 1, p.status, kErrAttnWait)) break;
        mbar_expect_tx(kv_full, 2 * kTile);
        load_tile(sK, &map_qkv, kv_full, (p.hq + hk) * kD, row0 + j * kBlk);
        load_tile(sV, &map_qkv, kv_full, (p.hq + p.hkv + hk) * kD, row0 + j * kBlk);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, p.status, kErrAttnWait);
      for (int j = 0; j < n_kv && ok; ++j) {
        ok = mbar_wait(kv_full, j & 1, p.status, kErrAttnWait);
        if (!ok) break;
        tc_fence_after_sync();
        mma_128<false, false>(tS, smem_u32(sQ), smem_u32(sK), false);    // S  = Q  K^T
        mma_128<false, false>(tdP, smem_u32(sdO), smem_u32(sV), false);  // dP = dO V^T
        tc_commit(sdp_full);
        ok = mbar_wait(ds_full, j & 1, p.status, kErrAttnWait);
        if (!ok) break;
        tc_fence_after_sync();
        mma_128<false, true>(tdQ, smem_u32(sdS), smem_u32(sK), j > 0);   // dQ += dS K
        tc_commit(kv_empty);
      }
      if (!ok) tc_commit(sdp_full);
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int q_idx = qb * kBlk + r;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const bool q_ok = q_idx < p.seq;
    const int64_t stat = (static_cast<int64_t>(b) * p.hq + h) * p.seq + min(q_idx, p.seq - 1);
    const float lse = p.lse[stat], dlt = p.delta[stat];
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      ok = mbar_wait(sdp_full, j & 1, p.status, kErrAttnWait);
      if (!ok) break;
      tc_fence_after_sync();
      const bool diag = (j == qb);
      uint32_t mw[4];
      load_key_bits(p.key_bits, p.bits_pitch, p.key_mask, p.seq, b, j, mw);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t s[32], d[32];
        tmem_ld_32x32(tS + lane_base + c * 32, s);
        tmem_ld_32x32(tdP + lane_base + c * 32, d);
        tmem_ld_wait();
        float ds[32];
        const uint32_t word = mw[c];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kv = j * kBlk + c * 32 + i;
          const bool keep = q_ok && (!diag || kv <= q_idx) && ((word >> i) & 1u);
          const float pr = keep ? __expf(__uint_as_float(s[i]) * p.scale - lse) : 0.f;
          ds[i] = pr * (__uint_as_float(d[i]) - dlt) * p.scale;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 pk;
          pk.x = pack_bf16x2(ds[8 * g], ds[8 * g + 1]);
          pk.y = pack_bf16x2(ds[8 * g + 2], ds[8 * g + 3]);
          pk.z = pack_bf16x2(ds[8 * g + 4], ds[8 * g + 5]);
          pk.w = pack_bf16x2(ds[8 * g + 6], ds[8 * g + 7]);
          store_row8(sdS, r, c * 4 + g, pk);
        }
      }
      tc_fence_before_sync();
      fence_proxy_async();
      mbar_arrive(ds_full);
    }
    // dQ is complete once the last dS K product has retired (kv_empty's last phase)
    if (ok) ok = mbar_wait(kv_empty, (n_kv - 1) & 1, p.status, kErrAttnWait);
    tc_fence_after_sync();
    __nv_bfloat16* drow = p.dqkv + static_cast<int64_t>(row0 + q_idx) * (p.hq + 2 * p.hkv) * kD + h * kD;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t v[32];
      tmem_ld_32x32(tdQ + lane_base + c * 32, v);
      tmem_ld_wait();
      if (ok && q_ok) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 pk;
          pk.x = pack_bf16x2(__uint_as_float(v[8 * g]), __uint_as_float(v[8 * g + 1]));
          pk.y = pack_bf16x2(__uint_as_float(v[8 * g + 2]), __uint_as_float(v[8 * g + 3]));
          pk.z = pack_bf16x2(__uint_as_float(v[8 * g + 4]), __uint_as_float(v[8 * g + 5]));
          pk.w = pack_bf16x2(__uint_as_float(v[8 * g + 6]), __uint_as_float(v[8 * g + 7]));
          *reinterpret_cast<uint4*>(drow + c * 32 + g * 8) = pk;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------- dK, dV
// One CTA per (key block j, kv head x part, batch); loops over its share of the query heads of the
// GQA group and the query blocks i >= j, so dK / dV accumulate in TMEM and are written once.
// With parts == 1 the CTA owns the whole group and writes bf16 dK / dV; with parts > 1 (small
// batches would otherwise leave most SMs idle) each part writes an fp32 partial plane and
// attention_dkv_finish_kernel adds the planes in a fixed order.
// Scores are formed transposed (rows = keys): S^T = K Q^T, dP^T = V dO^T, so each softmax thread
// owns one key row and writes P^T / dS^T rows directly as K-major operands of
//   dV += P^T dO,   dK += dS^T Q.
// smem: K | V | Q | dO | P^T | dS^T | lse[128] delta[128] | barriers
constexpr int kDkvSmem = 6 * kTile + 1024 + 1024 + 256;

__global__ void __launch_bounds__(kThreads, 1)
attention_dkv_kernel(const __grid_constant__ CUtensorMap map_qkv,
                     const __grid_constant__ CUtensorMap map_do, BwdParams p) {
  if (kernel_should_skip(p.status)) return;   // an earlier kernel already failed
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + kTile;
  uint8_t* sQ = sV + kTile;
  uint8_t* sdO = sQ + kTile;
  uint8_t* sPT = sdO + kTile;
  uint8_t* sdST = sPT + kTile;
  float* s_lse = reinterpret_cast<float*>(sdST + kTile);
  float* s_dlt = s_lse + 128;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_dlt + 128);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;
  uint64_t* q_empty = bars + 2;
  uint64_t* st_full = bars + 3;
  uint64_t* pt_full = bars + 4;   // 128 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb = blockIdx.x, hk = blockIdx.y / p.parts, part = blockIdx.y % p.parts, b = blockIdx.z;
  const int group = p.hq / p.hkv;
  const int heads_here = group / p.parts;   // parts divides group (checked on the host)
  const int head0 = hk * group + part * heads_here;
  const int n_q = (p.seq + kBlk - 1) / kBlk;
  const int per_head = n_q - kb;          // query blocks kb .. n_q-1
  const int iters = heads_here * per_head;
  const int row0 = b * p.seq;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    mbar_init(st_full, 1);
    mbar_init(pt_full, 128);
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tST = tmem, tdPT = tmem + 128, tdV = tmem + 256, tdK = tmem + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * kTile);
      load_tile(sK, &map_qkv, kv_full, (p.hq + hk) * kD, row0 + kb * kBlk);
      load_tile(sV, &map_qkv, kv_full, (p.hq + p.hkv + hk) * kD, row0 + kb * kBlk);
      for (int t = 0; t < iters; ++t) {
        const int h = head0 + t / per_head;
        const int i = kb + t % per_head;
        if (!mbar_wait(q_empty, (t & 1) ^ 1, p.status, kErrAttnWait)) break;
        mbar_expect_tx(q_full, 2 * kTile);
        load_tile(sQ, &map_qkv, q_full, h * kD, row0 + i * kBlk);
        load_tile(sdO, &map_do, q_full, h * kD, row0 + i * kBlk);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(kv_full, 0, p.status, kErrAttnWait);
      for (int t = 0; t < iters && ok; ++t) {
        ok = mbar_wait(q_full, t & 1, p.status, kErrAttnWait);
        if (!ok) break;
        tc_fence_after_sync();
        mma_128<false, false>(tST, smem_u32(sK), smem_u32(sQ), false);    // S^T  = K Q^T
        mma_128<false, false>(tdPT, smem_u32(sV), smem_u32(sdO), false);  // dP^T = V dO^T
        tc_commit(st_full);
        ok = mbar_wait(pt_full, t & 1, p.status, kErrAttnWait);
        if (!ok) break;
        tc_fence_after_sync();
        mma_128<false, true>(tdV, smem_u32(sPT), smem_u32(sdO), t > 0);   // dV += P^T dO
        mma_128<false, true>(tdK, smem_u32(sdST), smem_u32(sQ), t > 0);   // dK += dS^T Q
        tc_commit(q_empty);
      }
      if (!ok) tc_commit(st_full);
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;              // key row inside the tile
    const int kv_idx = kb * kBlk + r;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    bool kv_ok = kv_idx < p.seq;
    if (kv_ok && p.key_bits != nullptr)
      kv_ok = (p.key_bits[static_cast<int64_t>(b) * p.bits_pitch + (kv_idx >> 5)] >> (kv_idx & 31)) & 1u;
    else if (kv_ok && p.key_mask != nullptr)
      kv_ok = p.key_mask[b * p.seq + kv_idx] != 0;
    bool ok = true;
    for (int t = 0; t < iters; ++t) {
      const int h = head0 + t / per_head;
      const int i = kb + t % per_head;
      softmax_bar();  // everyone finished reading the previous block's lse / delta
      {
        const int qi = i * kBlk + r;
        const int64_t stat = (static_cast<int64_t>(b) * p.hq + h) * p.seq + min(qi, p.seq - 1);
        s_lse[r] = p.lse[stat];
        s_dlt[r] = p.delta[stat];
      }
      softmax_bar();
      // after a failed wait the loop keeps its shape (no early exit) so that every thread
      // still reaches the named barriers above the same number of times
      if (ok) ok = mbar_wait(st_full, t & 1, p.status, kErrAttnWait);
      tc_fence_after_sync();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t s[32], d[32];
        tmem_ld_32x32(tST + lane_base + c * 32, s);
        tmem_ld_32x32(tdPT + lane_base + c * 32, d);
        tmem_ld_wait();
        float pt[32], ds[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const int col = c * 32 + x;
          const int qi = i * kBlk + col;
          const bool keep = kv_ok && qi < p.seq && qi >= kv_idx;
          const float pr = keep ? __expf(__uint_as_float(s[x]) * p.scale - s_lse[col]) : 0.f;
          pt[x] = pr;
          ds[x] = pr * (__uint_as_float(d[x]) - s_dlt[col]) * p.scale;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 a, e;
          a.x = pack_bf16x2(pt[8 * g], pt[8 * g + 1]);
          a.y = pack_bf16x2(pt[8 * g + 2], pt[8 * g + 3]);
          a.z = pack_bf16x2(pt[8 * g + 4], pt[8 * g + 5]);
          a.w = pack_bf16x2(pt[8 * g + 6], pt[8 * g + 7]);
          e.x = pack_bf16x2(ds[8 * g], ds[8 * g + 1]);
          e.y = pack_bf16x2(ds[8 * g + 2], ds[8 * g + 3]);
          e.z = pack_bf16x2(ds[8 * g + 4], ds[8 * g + 5]);
          e.w = pack_bf16x2(ds[8 * g + 6], ds[8 * g + 7]);
          store_row8(sPT, r, c * 4 + g, a);
          store_row8(sdST, r, c * 4 + g, e);
        }
      }
      tc_fence_before_sync();
      fence_proxy_async();
      mbar_arrive(pt_full);
    }
    if (ok) ok = mbar_wait(q_empty, (iters - 1) & 1, p.status, kErrAttnWait);
    tc_fence_after_sync();
    const int64_t width = static_cast<int64_t>(p.hq + 2 * p.hkv) * kD;
    __nv_bfloat16* krow = p.dqkv + (row0 + kv_idx) * width + (p.hq + hk) * kD;
    __nv_bfloat16* vrow = krow + p.hkv * kD;
    const bool store = ok && kv_idx < p.seq;
    const int64_t pwidth = static_cast<int64_t>(2 * p.hkv) * kD;
    float* pk_row = p.parts > 1
                        ? p.dkv_part + (static_cast<int64_t>(part) * p.batch * p.seq + row0 + kv_idx) * pwidth +
                              hk * kD
                        : nullptr;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t dk[32], dv[32];
      tmem_ld_32x32(tdK + lane_base + c * 32, dk);
      tmem_ld_32x32(tdV + lane_base + c * 32, dv);
      tmem_ld_wait();
      if (store && p.parts > 1) {
        float* pv_row = pk_row + p.hkv * kD;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          *reinterpret_cast<uint4*>(pk_row + c * 32 + g * 4) =
              make_uint4(dk[4 * g], dk[4 * g + 1], dk[4 * g + 2], dk[4 * g + 3]);
          *reinterpret_cast<uint4*>(pv_row + c * 32 + g * 4) =
              make_uint4(dv[4 * g], dv[4 * g + 1], dv[4 * g + 2], dv[4 * g + 3]);
        }
      } else if (store) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 a, e;
          a.x = pack_bf16x2(__uint_as_float(dk[8 * g]), __uint_as_float(dk[8 * g + 1]));
          a.y = pack_bf16x2(__uint_as_float(dk[8 * g + 2]), __uint_as_float(dk[8 * g + 3]));
          a.z = pack_bf16x2(__uint_as_float(dk[8 * g + 4]), __uint_as_float(dk[8 * g + 5]));
          a.w = pack_bf16x2(__uint_as_float(dk[8 * g + 6]), __uint_as_float(dk[8 * g + 7]));
          e.x = pack_bf16x2(__uint_as_float(dv[8 * g]), __uint_as_float(dv[8 * g + 1]));
          e.y = pack_bf16x2(__uint_as_float(dv[8 * g + 2]), __uint_as_float(dv[8 * g + 3]));
          e.z = pack_bf16x2(__uint_as_float(dv[8 * g + 4]), __uint_as_float(dv[8 * g + 5]));
          e.w = pack_bf16x2(__uint_as_float(dv[8 * g + 6]), __uint_as_float(dv[8 * g + 7]));
          *reinterpret_cast<uint4*>(krow + c * 32 + g * 8) = a;
          *reinterpret_cast<uint4*>(vrow + c * 32 + g * 8) = e;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// dqkv[row, K|V columns] = bf16(sum over parts of the fp32 partial planes), fixed order.
__global__ void attention_dkv_finish_kernel(const float* __restrict__ part, int parts,
                                            int64_t rows, int hq, int hkv,
                                            __nv_bfloat16* __restrict__ dqkv) {
  const int64_t pwidth = static_cast<int64_t>(2 * hkv) * kD;     // floats per row of a plane
  const int64_t vec = pwidth / 8;
  const int64_t width = static_cast<int64_t>(hq + 2 * hkv) * kD;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < rows * vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / vec;
    const int64_t col = (i - row * vec) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < parts; ++k) {
      const float4* src = reinterpret_cast<const float4*>(part + (k * rows + row) * pwidth + col);
      const float4 a = src[0], b = src[1];
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    uint4 pk;
    pk.x = pack_bf16x2(acc[0], acc[1]);
    pk.y = pack_bf16x2(acc[2], acc[3]);
    pk.z = pack_bf16x2(acc[4], acc[5]);
    pk.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(dqkv + row * width + static_cast<int64_t>(hq) * kD + col) = pk;
  }
}

template <typename K>
cudaError_t opt_in_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

}  // namespace

cudaError_t launch_attention_fwd(const AttnCall& c, int* status, cudaStream_t s) {
  if (c.seq < 1 || c.hq % c.hkv) return cudaErrorInvalidValue;
  const int64_t rows = static_cast<int64_t>(c.batch) * c.seq;
  const int64_t width = static_cast<int64_t>(c.hq + 2 * c.hkv) * kD;
  CUtensorMap map;
  if (!make_bf16_tensor_map(&map, c.qkv, rows, width, width, 64, kBlk)) return cudaErrorInvalidValue;
  static cudaError_t attr = opt_in_smem(attention_fwd_kernel, kFwdSmem);
  if (attr != cudaSuccess) return attr;
  if (c.key_bits != nullptr &&
      (c.key_bits_pitch < 4 * ((c.seq + kBlk - 1) / kBlk) || (c.key_bits_pitch % 4) ||
       (reinterpret_cast<uintptr_t>(c.key_bits) & 15)))
    return cudaErrorInvalidValue;
  FwdParams p{reinterpret_cast<__nv_bfloat16*>(c.out), c.lse, c.key_mask, c.batch, c.seq, c.hq,
              c.hkv, c.scale, status, c.key_bits, c.key_bits_pitch};
  dim3 grid((c.seq + kBlk - 1) / kBlk, c.hq, c.batch);
  attention_fwd_kernel<<<grid, kThreads, kFwdSmem, s>>>(map, p);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_attention_bwd(const AttnBwdCall& c, int* status, cudaStream_t s) {
  if (c.seq < 1 || c.hq % c.hkv) return cudaErrorInvalidValue;
  const int64_t rows = static_cast<int64_t>(c.batch) * c.seq;
  const int64_t width = static_cast<int64_t>(c.hq + 2 * c.hkv) * kD;
  const int64_t owidth = static_cast<int64_t>(c.hq) * kD;
  CUtensorMap map_qkv, map_do;
  if (!make_bf16_tensor_map(&map_qkv, c.qkv, rows, width, width, 64, kBlk) ||
      !make_bf16_tensor_map(&map_do, c.dout, rows, owidth, owidth, 64, kBlk))
    return cudaErrorInvalidValue;
  static cudaError_t attr1 = opt_in_smem(attention_dq_kernel, kDqSmem);
  static cudaError_t attr2 = opt_in_smem(attention_dkv_kernel, kDkvSmem);
  if (attr1 != cudaSuccess) return attr1;
  if (attr2 != cudaSuccess) return attr2;
  const int64_t warps = rows * c.hq;
  attention_delta_kernel<<<static_cast<int>((warps * 32 + 255) / 256), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(c.out), reinterpret_cast<const __nv_bfloat16*>(c.dout),
      c.delta, c.batch, c.seq, c.hq);
  count_launch();
  const int nblk = (c.seq + kBlk - 1) / kBlk;
  int parts = 1;
  if (c.dkv_accum != nullptr) {
    parts = attention_bwd_parts(c.batch, c.seq, c.hq, c.hkv);
    const int64_t need = static_cast<int64_t>(parts) * rows * 2 * c.hkv * kD;
    if (parts > 1 && c.dkv_accum_floats < need) return cudaErrorInvalidValue;
  }
  if (c.key_bits != nullptr &&
      (c.key_bits_pitch < 4 * nblk || (c.key_bits_pitch % 4) ||
       (reinterpret_cast<uintptr_t>(c.key_bits) & 15)))
    return cudaErrorInvalidValue;
  BwdParams p{c.lse, c.delta, reinterpret_cast<__nv_bfloat16*>(c.dqkv), c.key_mask, c.batch, c.seq,
              c.hq, c.hkv, c.scale, status, parts > 1 ? c.dkv_accum : nullptr, parts,
              c.key_bits, c.key_bits_pitch};
  attention_dkv_kernel<<<dim3(nblk, c.hkv * parts, c.batch), kThreads, kDkvSmem, s>>>(map_qkv,
                                                                                     map_do, p);
  count_launch();
  attention_dq_kernel<<<dim3(nblk, c.hq, c.batch), kThreads, kDqSmem, s>>>(map_qkv, map_do, p);
  count_launch();
  if (parts > 1) {
    const int64_t work = rows * (2 * c.hkv * kD / 8);
    const int grid = static_cast<int>(std::min<int64_t>((work + 255) / 256, sm_count() * 8));
    attention_dkv_finish_kernel<<<grid, 256, 0, s>>>(c.dkv_accum, parts, rows, c.hq, c.hkv,
                                                     reinterpret_cast<__nv_bfloat16*>(c.dqkv));
    count_launch();
  }
  return cudaGetLastError();
}

namespace {
// bits[b, w] bit i = (mask[b, 32 w + i] != 0); words beyond the sequence are zero
__global__ void pack_key_mask_kernel(const uint8_t* __restrict__ mask, uint32_t* __restrict__ bits,
                                     int batch, int seq, int pitch) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= batch * pitch) return;
  const int b = idx / pitch, w = idx - b * pitch;
  uint32_t word = 0;
  for (int i = 0; i < 32; ++i) {
    const int kv = w * 32 + i;
    if (kv < seq && mask[static_cast<int64_t>(b) * seq + kv] != 0) word |= 1u << i;
  }
  bits[idx] = word;
}
}  // namespace

cudaError_t launch_pack_key_mask(const uint8_t* mask, uint32_t* bits, int batch, int seq, int pitch,
                                 cudaStream_t s) {
  if (batch < 1 || seq < 1 || pitch < 4 * ((seq + kBlk - 1) / kBlk) || (pitch % 4))
    return cudaErrorInvalidValue;
  const int total = batch * pitch;
  pack_key_mask_kernel<<<(total + 127) / 128, 128, 0, s>>>(mask, bits, batch, seq, pitch);
  count_launch();
  return cudaGetLastError();
}

int attention_bwd_parts(int batch, int seq, int hq, int hkv) {
  // smallest split of the query-head group that puts at least one dK/dV CTA on every SM
  const int group = hq / hkv;
  const int nblk = (seq + kBlk - 1) / kBlk;
  const int base = nblk * hkv * batch;
  for (int parts = 1; parts <= group; ++parts)
    if (group % parts == 0 && base * parts >= sm_count()) return parts;
  return group;
}

}  // namespace stb
