// Collectives written as kernels over NVLink peer memory (plain P2P loads through NVSwitch), each
// fused with the compute that follows it in the reference's NCCL pipeline:
//   * parameter all-gather + copy-out + fp32->bf16 cast  (src/sharded_runtime/runtime/materializer.py:31-114,
//     src/sharded_runtime/runtime/layout.py:77-90)
//   * gradient pack + reduce-scatter + 1/F scale + accumulate (+ AdamW)  (materializer.py:116-192,
//     layout.py:93-106, src/sharded_runtime/training/qwen2_trainer.py:48); with a multicast
//     address of the gradient slots the sum over the FSDP members is one `multimem.ld_reduce`
//     per 16 bytes, carried out inside the NVSwitch
//   * sequence-parallel activation gather / reduce-scatter (src/sharded_runtime/runtime/comm.py:781-884)
//   * embedding rows fetched from the owning shard without gathering the table.
// With degree 1 the same kernels read only local memory.  No kernel here waits on another GPU
// except the flag barrier and the small all-reduce, whose waits are bounded in time.
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>

#include "api.h"
#include "common.cuh"

namespace stb {

namespace {

constexpr int kMaxSegs = 32;
struct SegTable {
  SegmentDesc s[kMaxSegs];
  int n;
};

__device__ __forceinline__ uint32_t pk2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Work is tiled in chunks of kChunk elements of one segment; blockIdx.y = segment.
constexpr int kChunk = 4096;

struct ShadowPtrs {
  const __nv_bfloat16* p[kMaxPeers];
};

// bf16 -> bf16 gather of one segment from the owners' compute-dtype shadow shards: the cast
// already happened where the optimizer wrote the parameter, so only 2 bytes per element cross
// NVLink instead of 4 (rounding before or after the transfer gives the same bits).
constexpr int kChunkB = 8192;
__device__ __forceinline__ void gather_shadow_segment(const ShadowPtrs& sh, const SegmentDesc& sg,
                                                      __nv_bfloat16* __restrict__ full_bf16) {
  const bool vec = (sg.q % 8 == 0) && (sg.shard_off % 8 == 0) && (sg.full_off % 8 == 0);
  for (int64_t chunk = blockIdx.x; chunk * kChunkB < sg.numel; chunk += gridDim.x) {
    const int64_t base = chunk * kChunkB;
    if (vec && base + kChunkB <= sg.numel && blockDim.x * 8 * 4 == kChunkB) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t i = base + (u * blockDim.x + threadIdx.x) * 8;
        const int r = static_cast<int>(i / sg.q);
        v[u] = *reinterpret_cast<const uint4*>(sh.p[r] + sg.shard_off + (i - r * sg.q));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t i = base + (u * blockDim.x + threadIdx.x) * 8;
        *reinterpret_cast<uint4*>(full_bf16 + sg.full_off + i) = v[u];
      }
    } else {
      const int64_t end = min(base + kChunkB, sg.numel);
      if (vec) {
        for (int64_t i = base + threadIdx.x * 8; i < end; i += blockDim.x * 8) {
          const int r = static_cast<int>(i / sg.q);
          const __nv_bfloat16* src = sh.p[r] + sg.shard_off + (i - r * sg.q);
          if (i + 7 < sg.numel) {
            *reinterpret_cast<uint4*>(full_bf16 + sg.full_off + i) =
                *reinterpret_cast<const uint4*>(src);
          } else {
            for (int64_t j = i; j < sg.numel; ++j) full_bf16[sg.full_off + j] = src[j - i];
          }
        }
      } else {
        for (int64_t i = base + threadIdx.x; i < end; i += blockDim.x) {
          const int r = static_cast<int>(i / sg.q);
          full_bf16[sg.full_off + i] = sh.p[r][sg.shard_off + (i - r * sg.q)];
        }
      }
    }
  }
}

__global__ void gather_params_kernel(PeerPtrs shards, ShadowPtrs shadows, int use_shadow, int degree,
                                     SegTable tab, __nv_bfloat16* __restrict__ full_bf16,
                                     float* __restrict__ full_fp32) {
  const SegmentDesc sg = tab.s[blockIdx.y];
  if (use_shadow && !sg.keep_fp32) {
    gather_shadow_segment(shadows, sg, full_bf16);
    return;
  }
  const bool vec = (sg.q % 4 == 0) && (sg.shard_off % 4 == 0) && (sg.full_off % 4 == 0);
  for (int64_t chunk = blockIdx.x; chunk * kChunk < sg.numel; chunk += gridDim.x) {
    const int64_t base = chunk * kChunk;
    if (vec && base + kChunk <= sg.numel && blockDim.x * 4 * 4 == kChunk) {
      // full chunk: four independent 16-byte loads in flight per thread before any store
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t i = base + (u * blockDim.x + threadIdx.x) * 4;
        const int r = static_cast<int>(i / sg.q);
        v[u] = *reinterpret_cast<const float4*>(shards.p[r] + sg.shard_off + (i - r * sg.q));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t i = base + (u * blockDim.x + threadIdx.x) * 4;
        if (sg.keep_fp32) {
          *reinterpret_cast<float4*>(full_fp32 + sg.full_off + i) = v[u];
        } else {
          uint2 o;
          o.x = pk2(v[u].x, v[u].y);
          o.y = pk2(v[u].z, v[u].w);
          *reinterpret_cast<uint2*>(full_bf16 + sg.full_off + i) = o;
        }
      }
    } else if (vec) {
      for (int64_t i = base + threadIdx.x * 4; i < min(base + kChunk, sg.numel);
           i += blockDim.x * 4) {
        const int r = static_cast<int>(i / sg.q);  // q % 4 == 0: the 4 elements share a rank
        const int64_t off = i - r * sg.q;
        const float* src = shards.p[r] + sg.shard_off + off;
        if (i + 3 < sg.numel) {
          const float4 v = *reinterpret_cast<const float4*>(src);
          if (sg.keep_fp32) {
            *reinterpret_cast<float4*>(full_fp32 + sg.full_off + i) = v;
          } else {
            uint2 o;
            o.x = pk2(v.x, v.y);
            o.y = pk2(v.z, v.w);
            *reinterpret_cast<uint2*>(full_bf16 + sg.full_off + i) = o;
          }
        } else {
          for (int64_t j = i; j < sg.numel; ++j) {
            const float v = src[j - i];
            if (sg.keep_fp32)
              full_fp32[sg.full_off + j] = v;
            else
              full_bf16[sg.full_off + j] = __float2bfloat16(v);
          }
        }
      }
    } else {
      for (int64_t i = base + threadIdx.x; i < min(base + kChunk, sg.numel); i += blockDim.x) {
        const int r = static_cast<int>(i / sg.q);
        const float v = shards.p[r][sg.shard_off + (i - r * sg.q)];
        if (sg.keep_fp32)
          full_fp32[sg.full_off + i] = v;
        else
          full_bf16[sg.full_off + i] = __float2bfloat16(v);
      }
    }
  }
}

// Rank `rank` owns elements [rank*q, rank*q + q) of each segment (zero beyond numel).
// With a tensor-parallel axis (tp > 1) `full` lists the gradient slots of the whole mesh in rank
// order (index f * tp + t).  A TP-split parameter is summed over the F ranks of this rank's TP
// coordinate; a TP-replicated one (segment flag `pad`) over all F * tp ranks, scaled by
// rep_scale -- the T-way sum that the reference issues as a separate all-reduce after its
// reduce-scatter (src/sharded_runtime/runtime/materializer.py:228-233).
template <bool ADAMW>
__global__ void reduce_scatter_kernel(PeerPtrs full, int degree, int rank, int tp, int tp_rank,
                                      SegTable tab, float* __restrict__ gshard,
                                      float* __restrict__ p, float* __restrict__ m,
                                      float* __restrict__ v, float split_scale, float rep_scale,
                                      int accumulate, AdamWArgs a, int* __restrict__ flags,
                                      __nv_bfloat16* __restrict__ shadow, const int* status,
                                      const float* __restrict__ multicast) {
  // A failure recorded earlier (a peer that never signalled) means the slots may hold stale
  // data: neither the gradient shard nor, with ADAMW, the parameters are touched.
  if (kernel_should_skip(status)) return;
  const SegmentDesc sg = tab.s[blockIdx.y];
  const bool replicated = tp > 1 && sg.pad != 0;
  const int n_src = replicated ? degree * tp : degree;
  // replicated segments use one fixed summation order so every TP replica computes bit-identical
  // shard gradients (and updates); split segments rotate the order to spread the load
  const int first = replicated ? 0 : rank;
  const int stride = replicated ? 1 : tp;
  const int offset = replicated ? 0 : tp_rank;
  const float scale = replicated ? rep_scale : split_scale;
  const int64_t lo = static_cast<int64_t>(rank) * sg.q;
  const int64_t valid = max(static_cast<int64_t>(0), min(sg.q, sg.numel - lo));
  const bool vec = (sg.q % 4 == 0) && (sg.shard_off % 4 == 0) && (sg.full_off % 4 == 0);
  const float step_size = ADAMW ? a.lr / a.bias_correction1 : 0.f;
  const float inv_bc2_sqrt = ADAMW ? rsqrtf(a.bias_correction2) : 0.f;
  // the gradient check rides along: flags[0] = a non-finite reduced gradient was written,
  // flags[1] = a padding element of the shard is not exactly zero
  int bad = 0, pad_bad = 0;
  for (int64_t chunk = blockIdx.x; chunk * kChunk < sg.q; chunk += gridDim.x) {
    const int64_t base = chunk * kChunk;
    const int64_t end = min(base + kChunk, sg.q);
    const int step = vec ? 4 : 1;
    for (int64_t i = base + threadIdx.x * step; i < end; i += blockDim.x * step) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const int cnt = vec ? 4 : 1;
      if (vec && i + 3 < valid && multicast != nullptr && !replicated) {
        // NVLS: one load through the multicast address of the gradient slot; the NVSwitch reads
        // the same 16 bytes of every member's slot, adds them and returns the sum, so only
        // 1 / F of the gradient enters this GPU instead of (F - 1) / F
        float4 t;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(t.x), "=f"(t.y), "=f"(t.z), "=f"(t.w)
                     : "l"(multicast + sg.full_off + lo + i)
                     : "memory");
        acc[0] = t.x; acc[1] = t.y; acc[2] = t.z; acc[3] = t.w;
      } else if (vec && i + 3 < valid) {
        // rotate the peer order by rank so the ranks do not all hit one peer at once
        for (int d = 0; d < n_src; ++d) {
          const int src = ((first + d) % n_src) * stride + offset;
          const float4 t =
              *reinterpret_cast<const float4*>(full.p[src] + sg.full_off + lo + i);
          acc[0] += t.x; acc[1] += t.y; acc[2] += t.z; acc[3] += t.w;
        }
      } else {
        for (int j = 0; j < cnt; ++j) {
          if (i + j < valid) {
            for (int d = 0; d < n_src; ++d) {
              const int src = ((first + d) % n_src) * stride + offset;
              acc[j] += full.p[src][sg.full_off + lo + i + j];
            }
          }
        }
      }
      if (vec) {
        // q % 4 == 0: the four elements are inside the shard; 16-byte accesses throughout
        const int64_t e = sg.shard_off + i;
        float4 g = make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
        if (accumulate) {
          const float4 o = *reinterpret_cast<const float4*>(gshard + e);
          g.x += o.x; g.y += o.y; g.z += o.z; g.w += o.w;
        }
        *reinterpret_cast<float4*>(gshard + e) = g;   // padding stays exactly zero: acc is 0 there
        bad |= !(isfinite(g.x) && isfinite(g.y) && isfinite(g.z) && isfinite(g.w));
        if (i + 3 >= valid) {
          const float* gp = &g.x;
          for (int j = 0; j < 4; ++j)
            if (i + j >= valid && gp[j] != 0.f) pad_bad = 1;
        }
        if (ADAMW) {
          float4 pv = *reinterpret_cast<const float4*>(p + e);
          float4 mv = *reinterpret_cast<const float4*>(m + e);
          float4 vv = *reinterpret_cast<const float4*>(v + e);
          float* pp = &pv.x; float* mp = &mv.x; float* vp = &vv.x; const float* gp = &g.x;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float gr = gp[j] * a.grad_scale;
            pp[j] *= 1.f - a.lr * a.weight_decay;
            mp[j] = a.beta1 * mp[j] + (1.f - a.beta1) * gr;
            vp[j] = a.beta2 * vp[j] + (1.f - a.beta2) * gr * gr;
            pp[j] -= step_size * mp[j] / (sqrtf(vp[j]) * inv_bc2_sqrt + a.eps);
          }
          *reinterpret_cast<float4*>(p + e) = pv;   // padding has p = g = m = v = 0 and stays 0
          if (shadow != nullptr) {                   // compute-dtype copy for the next gather
            uint2 pk;
            pk.x = pk2(pv.x, pv.y);
            pk.y = pk2(pv.z, pv.w);
            *reinterpret_cast<uint2*>(shadow + e) = pk;
          }
          *reinterpret_cast<float4*>(m + e) = mv;
          *reinterpret_cast<float4*>(v + e) = vv;
        }
      } else {
        const int64_t e = sg.shard_off + i;
        float g = acc[0] * scale;
        if (accumulate) g += gshard[e];
        gshard[e] = g;
        bad |= !isfinite(g);
        if (i >= valid && g != 0.f) pad_bad = 1;
        if (ADAMW) {
          float pj = p[e] * (1.f - a.lr * a.weight_decay);
          const float gr = g * a.grad_scale;
          const float mj = a.beta1 * m[e] + (1.f - a.beta1) * gr;
          const float vj = a.beta2 * v[e] + (1.f - a.beta2) * gr * gr;
          pj -= step_size * mj / (sqrtf(vj) * inv_bc2_sqrt + a.eps);
          p[e] = pj;
          m[e] = mj;
          v[e] = vj;
          if (shadow != nullptr) shadow[e] = __float2bfloat16(pj);
        }
      }
    }
  }
  if (flags != nullptr) {
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(&flags[0], 1);
    if (__syncthreads_or(pad_bad) && threadIdx.x == 0) atomicOr(&flags[1], 1);
  }
}

__global__ void embedding_gather_sharded_kernel(PeerPtrs shards, int degree, int64_t q,
                                                const int64_t* __restrict__ ids,
                                                float* __restrict__ out, int cols) {
  const int64_t row = blockIdx.x;
  const int64_t id = ids[row];
  const int64_t base = id * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const int64_t g = base + c;
    const int r = static_cast<int>(g / q);
    out[row * cols + c] = shards.p[r][g - r * q];
  }
}

struct VoidPeers {
  const void* p[kMaxPeers];
};

// out[b, r*sl + s, :] = peer r's x[b, s, :]   (16-byte vectors)
__global__ void seq_gather_kernel(VoidPeers peers, int degree, uint4* __restrict__ out, int batch,
                                  int seq_local, int64_t row_vec) {
  const int64_t per_peer = static_cast<int64_t>(batch) * seq_local * row_vec;
  const int64_t per_batch = seq_local * row_vec;
  const int64_t total = per_peer * degree;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // four independent 16-byte loads in flight per thread: remote latency is several microseconds
  for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total;
       i0 += 4 * stride) {
    uint4 v[4];
    int64_t dst[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t i = i0 + u * stride;
      dst[u] = -1;
      if (i < total) {
        const int r = static_cast<int>(i / per_peer);
        const int64_t j = i - r * per_peer;
        const int64_t b = j / per_batch;
        v[u] = reinterpret_cast<const uint4*>(peers.p[r])[j];
        dst[u] = (b * degree + r) * per_batch + (j - b * per_batch);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (dst[u] >= 0) out[dst[u]] = v[u];
  }
}

struct FloatPeers {
  const float* p[kMaxPeers];
};

// out[b, s, :] = residual[b, s, :] + sum_r partial_r[b, rank*sl + s, :]
__global__ void seq_reduce_scatter_kernel(FloatPeers peers, int degree, int rank,
                                          const float* __restrict__ residual,
                                          float* __restrict__ out, int batch, int seq_local,
                                          int cols) {
  const int64_t cv = cols / 4;
  const int64_t total = static_cast<int64_t>(batch) * seq_local * cv;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t b = i / (seq_local * cv);
    const int64_t rest = i - b * seq_local * cv;
    const int64_t src = (b * degree + rank) * seq_local * cv + rest;
    float4 acc = residual ? reinterpret_cast<const float4*>(residual)[i]
                          : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int d = 0; d < degree; ++d) {
      const int r = (rank + d) % degree;
      const float4 t = reinterpret_cast<const float4*>(peers.p[r])[src];
      acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
    }
    reinterpret_cast<float4*>(out)[i] = acc;
  }
}

struct FlagPeers {
  uint32_t* p[kMaxPeers];
};

// First expiry wins the status block: {code, silent peer, epoch waited for, epoch last seen}.
__device__ __forceinline__ void report_flag_timeout(int* status, int peer, uint32_t expected,
                                                    const uint32_t* flag) {
  if (atomicCAS(status, kOk, kErrPeerFlagWait) == kOk) {
    status[1] = peer;
    status[2] = static_cast<int>(expected);
    status[3] = static_cast<int>(*reinterpret_cast<const volatile uint32_t*>(flag));
  }
}

// Bounded wait for `*flag` to reach `epoch` (epochs only grow; the signed distance tolerates
// wrap-around).  The bound is a time budget read from the global nanosecond timer; the wait also
// ends as soon as the status word shows that something already failed.  Returns true when seen.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, const int* status,
                                          uint64_t budget_ns) {
  uint32_t v;
  for (int i = 0; i < 64; ++i) {   // the common case: the peer is already there or nearly so
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int32_t>(v - epoch) >= 0) return true;
  }
  const uint64_t t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 32; ++i) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (static_cast<int32_t>(v - epoch) >= 0) return true;
      __nanosleep(64);
    }
    if (status_failed(status)) return false;
    if (global_ns() - t0 > budget_ns) return false;
  }
}

// Thread t tells peer t "rank `rank` reached `epoch`" and then waits until peer t says the same.
// Pad layout: pad[slot * kMaxPeers + source_rank].  The wait is bounded in time; on expiry the
// status block is set and the kernel returns.  When a failure is already recorded on entry the
// kernel still publishes its own epoch (so that healthy peers are not held up by this rank) but
// does not wait: after one silent peer the barriers queued behind it return at once.
__global__ void peer_barrier_kernel(FlagPeers pads, int degree, int rank, uint32_t epoch, int slot,
                                    int* status, uint64_t budget_ns) {
  const int t = threadIdx.x;
  if (t >= degree) return;
  const bool failed_before = status_failed(status);
  __threadfence_system();
  uint32_t* remote = pads.p[t] + slot * kMaxPeers + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  if (failed_before) return;
  const uint32_t* mine = pads.p[rank] + slot * kMaxPeers + t;
  const bool seen = wait_flag(mine, epoch, status, budget_ns);
  if (!seen && status != nullptr) report_flag_timeout(status, t, epoch, mine);
  __threadfence_system();
}

// Small all-reduce (at most kMetricWidth doubles) in one kernel: thread t pushes this rank's
// vector into peer t's inbox and publishes the epoch, waits (bounded) for peer t's epoch, then
// the first n threads combine the inbox rows in rank order -- every rank computes the same bits.
// Element i is a SUM, or a MIN when bit i of min_mask is set.  Inboxes are double buffered on
// the epoch's parity: a rank can run at most one reduction ahead of its slowest peer.
// Inbox layout: [2][kMaxPeers][kMetricWidth] doubles.
constexpr int kMetricWidth = 16;
struct InboxPeers {
  double* p[kMaxPeers];
};

__global__ void peer_allreduce_small_kernel(FlagPeers pads, InboxPeers inboxes, int degree, int rank,
                                            uint32_t epoch, int slot, const double* __restrict__ in,
                                            double* __restrict__ out, int n, uint32_t min_mask,
                                            int* status, uint64_t budget_ns) {
  const int t = threadIdx.x;
  const int parity = static_cast<int>(epoch & 1u);
  if (t < degree) {
    const bool failed_before = status_failed(status);
    double* dst = inboxes.p[t] + (static_cast<int64_t>(parity) * kMaxPeers + rank) * kMetricWidth;
    for (int i = 0; i < n; ++i) dst[i] = in[i];
    __threadfence_system();
    uint32_t* remote = pads.p[t] + slot * kMaxPeers + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    if (!failed_before) {
      const uint32_t* mine = pads.p[rank] + slot * kMaxPeers + t;
      const bool seen = wait_flag(mine, epoch, status, budget_ns);
      if (!seen && status != nullptr) report_flag_timeout(status, t, epoch, mine);
    }
    __threadfence_system();
  }
  __syncthreads();
  if (t < n) {
    const volatile double* rows =
        inboxes.p[rank] + static_cast<int64_t>(parity) * kMaxPeers * kMetricWidth;
    double acc = rows[t];
    for (int r = 1; r < degree; ++r) {
      const double v = rows[r * kMetricWidth + t];
      acc = ((min_mask >> t) & 1u) ? fmin(acc, v) : acc + v;
    }
    out[t] = acc;
  }
}

bool fill_table(SegTable* t, const SegmentDesc* segs, int n) {
  if (n < 1 || n > kMaxSegs) return false;
  for (int i = 0; i < n; ++i) t->s[i] = segs[i];
  t->n = n;
  return true;
}

int g_ctas_per_sm = 0;   // 0: read STB_COLLECTIVE_CTAS_PER_SM once (default below)
int chunks_for(const SegmentDesc* segs, int n, bool per_shard) {
  if (g_ctas_per_sm == 0) {
    const char* env = getenv("STB_COLLECTIVE_CTAS_PER_SM");
    g_ctas_per_sm = env != nullptr ? std::max(1, atoi(env)) : 48;   // measured: 8..48 equal, 4 slower
  }
  const int kCtasPerSm = g_ctas_per_sm;
  // grid.x of a (chunks, segments) grid.  The kernels loop over chunks, so the grid only has to
  // be large enough to keep the memory system busy; STB_COLLECTIVE_CTAS_PER_SM bounds the total
  // (CTAs per SM over all segments).  The compute stream has the higher priority, so a larger
  // grid does not keep GEMMs launched meanwhile from being placed.
  int64_t most = 1;
  for (int i = 0; i < n; ++i) {
    const int64_t len = per_shard ? segs[i].q : segs[i].numel;
    most = std::max<int64_t>(most, (len + kChunk - 1) / kChunk);
  }
  const int64_t budget = std::max<int64_t>(1, (sm_count() * kCtasPerSm) / std::max(1, n));
  // and never more than four CTAs per SM for one segment: more only adds scheduling work
  return static_cast<int>(std::min<int64_t>({most, budget, static_cast<int64_t>(sm_count() * 4)}));
}

}  // namespace

cudaError_t launch_gather_params(PeerPtrs shards, int degree, const SegmentDesc* segs, int n_segs,
                                 void* full_bf16, float* full_fp32, int64_t total_full,
                                 cudaStream_t s, const void* const* shadows) {
  (void)total_full;
  SegTable tab;
  if (degree < 1 || degree > kMaxPeers || !fill_table(&tab, segs, n_segs))
    return cudaErrorInvalidValue;
  ShadowPtrs sh{};
  if (shadows != nullptr)
    for (int i = 0; i < degree; ++i) {
      if (shadows[i] == nullptr || (reinterpret_cast<uintptr_t>(shadows[i]) & 15))
        return cudaErrorInvalidValue;
      sh.p[i] = reinterpret_cast<const __nv_bfloat16*>(shadows[i]);
    }
  dim3 grid(chunks_for(segs, n_segs, false), n_segs);
  gather_params_kernel<<<grid, 256, 0, s>>>(shards, sh, shadows != nullptr ? 1 : 0, degree, tab,
                                            reinterpret_cast<__nv_bfloat16*>(full_bf16), full_fp32);
  count_launch();
  return cudaGetLastError();
}

bool valid_mesh(int degree, int rank, TpAxis tp) {
  return degree >= 1 && tp.degree >= 1 && degree * tp.degree <= kMaxPeers && rank >= 0 &&
         rank < degree && tp.rank >= 0 && tp.rank < tp.degree;
}

cudaError_t launch_reduce_scatter_grads(PeerPtrs full_grads, int degree, int rank,
                                        const SegmentDesc* segs, int n_segs, float* grad_shard,
                                        int64_t shard_total, float scale, bool accumulate,
                                        int* flags, cudaStream_t s, TpAxis tp, const int* status,
                                        const float* multicast) {
  (void)shard_total;
  SegTable tab;
  if (!valid_mesh(degree, rank, tp) || !fill_table(&tab, segs, n_segs) ||
      (reinterpret_cast<uintptr_t>(multicast) & 15))
    return cudaErrorInvalidValue;
  dim3 grid(chunks_for(segs, n_segs, true), n_segs);
  reduce_scatter_kernel<false><<<grid, 256, 0, s>>>(
      full_grads, degree, rank, tp.degree, tp.rank, tab, grad_shard, nullptr, nullptr, nullptr,
      scale, tp.replicated_scale, accumulate ? 1 : 0, AdamWArgs{}, flags, nullptr, status,
      multicast);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_reduce_scatter_adamw(PeerPtrs full_grads, int degree, int rank,
                                        const SegmentDesc* segs, int n_segs, float* grad_shard,
                                        float* p, float* m, float* v, int64_t shard_total,
                                        float scale, bool accumulate, AdamWArgs a, int* flags,
                                        cudaStream_t s, TpAxis tp, void* shadow, const int* status,
                                        const float* multicast) {
  (void)shard_total;
  SegTable tab;
  if (!valid_mesh(degree, rank, tp) || !fill_table(&tab, segs, n_segs) ||
      (reinterpret_cast<uintptr_t>(multicast) & 15))
    return cudaErrorInvalidValue;
  dim3 grid(chunks_for(segs, n_segs, true), n_segs);
  reduce_scatter_kernel<true><<<grid, 256, 0, s>>>(
      full_grads, degree, rank, tp.degree, tp.rank, tab, grad_shard, p, m, v, scale,
      tp.replicated_scale, accumulate ? 1 : 0, a, flags,
      reinterpret_cast<__nv_bfloat16*>(shadow), status, multicast);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_embedding_gather_sharded(PeerPtrs shards, int degree, int64_t q,
                                            const int64_t* ids, float* out, int rows, int cols,
                                            cudaStream_t s) {
  if (degree < 1 || degree > kMaxPeers || q < 1) return cudaErrorInvalidValue;
  embedding_gather_sharded_kernel<<<rows, 256, 0, s>>>(shards, degree, q, ids, out, cols);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_seq_gather(const void* const* peers, int degree, void* out, int batch,
                              int seq_local, int64_t row_bytes, cudaStream_t s) {
  if (degree < 1 || degree > kMaxPeers || row_bytes % 16) return cudaErrorInvalidValue;
  VoidPeers vp;
  for (int i = 0; i < degree; ++i) vp.p[i] = peers[i];
  const int64_t total = static_cast<int64_t>(batch) * seq_local * (row_bytes / 16) * degree;
  const int grid = static_cast<int>(std::min<int64_t>((total + 1023) / 1024, sm_count() * 8));
  seq_gather_kernel<<<grid, 256, 0, s>>>(vp, degree, reinterpret_cast<uint4*>(out), batch,
                                         seq_local, row_bytes / 16);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_seq_reduce_scatter_f32(const float* const* peers, int degree, int rank,
                                          const float* residual, float* out, int batch,
                                          int seq_local, int cols, cudaStream_t s) {
  if (degree < 1 || degree > kMaxPeers || cols % 4) return cudaErrorInvalidValue;
  FloatPeers fp;
  for (int i = 0; i < degree; ++i) fp.p[i] = peers[i];
  const int64_t total = static_cast<int64_t>(batch) * seq_local * (cols / 4);
  const int grid = static_cast<int>(std::min<int64_t>((total + 255) / 256, sm_count() * 8));
  seq_reduce_scatter_kernel<<<grid, 256, 0, s>>>(fp, degree, rank, residual, out, batch, seq_local,
                                                 cols);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_peer_allreduce_small(uint32_t* const* flag_pads, double* const* inboxes, int degree,
                                        int rank, uint32_t epoch, int slot, const double* in,
                                        double* out, int n, uint32_t min_mask, int* status,
                                        uint64_t budget_ns, cudaStream_t s) {
  if (degree < 1 || degree > kMaxPeers || rank < 0 || rank >= degree || n < 1 || n > kMetricWidth)
    return cudaErrorInvalidValue;
  FlagPeers fp;
  InboxPeers ip;
  for (int i = 0; i < degree; ++i) {
    fp.p[i] = flag_pads[i];
    ip.p[i] = inboxes[i];
  }
  peer_allreduce_small_kernel<<<1, 32, 0, s>>>(fp, ip, degree, rank, epoch, slot, in, out, n,
                                               min_mask, status, budget_ns);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_peer_barrier(uint32_t* const* flag_pads, int degree, int rank, uint32_t epoch,
                                int slot, int* status, uint64_t budget_ns, cudaStream_t s) {
  if (degree < 1 || degree > kMaxPeers || rank < 0 || rank >= degree)
    return cudaErrorInvalidValue;
  FlagPeers fp;
  for (int i = 0; i < degree; ++i) fp.p[i] = flag_pads[i];
  peer_barrier_kernel<<<1, 32, 0, s>>>(fp, degree, rank, epoch, slot, status, budget_ns);
  count_launch();
  return cudaGetLastError();
}

}  // namespace stb
