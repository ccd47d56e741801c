// Host-side launch API of the sm_100a kernels (plain C++; no torch headers).
// bindings.cpp wraps these as torch custom ops; every function enqueues on `stream` and returns
// the CUDA error of the launch, never synchronising the device.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace stb {

// Streaming multiprocessors of the current device (queried once per process; grids are sized from
// it instead of from a constant).
int sm_count();
// Every kernel launch site of this library counts itself: the number of kernels launched by this
// process so far (benchmarks report the difference over their timed region).
void count_launch();
void count_launches(int64_t n);   // a replayed graph of n kernels
int64_t launches_total();

// ------------------------------------------------------------------ GEMM (gemm_sm100.cu)
struct GemmCall {
  const void* a;      // bf16; K-major: [M, lda] ; MN-major: [K, lda]
  const void* b;      // bf16; K-major: [N, ldb] ; MN-major: [K, ldb]
  void* out;          // bf16 or fp32 [M, ldo]
  const float* bias;  // optional fp32 [N]
  const void* residual;  // optional, dtype/ld of out
  int M, N, K;
  int64_t lda, ldb, ldo;
  bool a_mn, b_mn;
  bool out_fp32;
  bool accumulate;
  float alpha;
  int force_bn;  // 0 = rule, else 128, 192 or 256
  int split_k;   // K-split of the tail wave's tiles: 0 = rule, 1 = never, n = exactly n
  // 0 = plain outputs leave through TMA stores staged in shared memory when the output's base
  // and pitch allow it; -1 = always the per-thread row stores
  int staged_store;
  // Gated (SwiGLU) forward: b = fused [2 * gated_inter, K] gate|up weight (K-major), out = [M, 2 *
  // gated_inter] bf16 (gate|up), gated_out = [M, gated_inter] bf16 = silu(gate) * up.  N must be
  // 2 * gated_inter.
  void* gated_out;
  int gated_inter;
  // Optional sequence scatter of an fp32 result (see GemmEpilogue): row b*seq + s is written to
  // scatter_out[s / seq_local] at row b*seq_local + s % seq_local; `out` is then unused.
  float* scatter_out[8];
  int scatter_degree;  // 0 or 1: plain output
  int scatter_seq;
  int scatter_seq_local;
  int scatter_broadcast;  // 1: store every row into all scatter_out buffers (all-reduce push)
  // Optional sequence all-gather of the A operand inside the GEMM (pull_degree > 1, a K-major):
  // `a` is then the local [M, lda] buffer the kernel *fills* -- row b * (degree * seq_local) +
  // r * seq_local + s comes from row b * seq_local + s of pull_peers[r] (row pitch pull_src_ld
  // elements; peer pointers allowed, read with plain loads) -- and consumes tile by tile as the
  // rows land.  M must equal pull_batch * pull_degree * pull_seq_local.  The gathered rows stay
  // in `a` for later GEMMs.  One such GEMM at a time per device.
  const void* pull_peers[8];
  int pull_degree;
  int pull_batch;
  int pull_seq_local;
  int64_t pull_src_ld;
};
cudaError_t launch_gemm_bf16(const GemmCall& c, int* status, cudaStream_t stream);

// ------------------------------------------------------------------ elementwise (elementwise.cu)
cudaError_t launch_rmsnorm_fwd(const float* x, const float* w, void* y, float* inv, int rows,
                               int cols, float eps, bool y_fp32, cudaStream_t s);
// sum_out = residual (optional) + sum of n_slots fp32 [rows, cols] slots spaced slot_stride
// elements apart; with w: y = bf16 rmsnorm(sum_out) * w and inv = per-row inverse RMS.
cudaError_t launch_slot_sum_rmsnorm(const float* slots, int n_slots, int64_t slot_stride,
                                    const float* residual, float* sum_out, const float* w, void* y,
                                    float* inv, int rows, int cols, float eps, cudaStream_t s);
// dx_out = dres_in (optional) + rmsnorm backward of dy ; dw_partial [blocks, cols]
cudaError_t launch_rmsnorm_bwd(const float* dy, const float* x, const float* w, const float* inv,
                               const float* dres_in, float* dx_out, float* dw_partial,
                               int partial_rows, int rows, int cols, cudaStream_t s);
cudaError_t launch_colsum_f32(const float* partial, float* out, int rows, int cols,
                              bool accumulate, cudaStream_t s);
cudaError_t launch_colsum_bf16(const void* x, int64_t ldx, float* out, int rows, int cols,
                               bool accumulate, float* scratch, int scratch_rows, cudaStream_t s);
// In-place rotary embedding on the q and k heads of a packed [rows, (hq + 2 hkv) * d] bf16 buffer.
cudaError_t launch_rope(void* qkv, const float* cos, const float* sin, const int* positions,
                        int rows, int seq, int hq, int hkv, int d, bool inverse, cudaStream_t s);
cudaError_t launch_swiglu_fwd(const void* gu, void* h, int rows, int inter, cudaStream_t s);
cudaError_t launch_swiglu_bwd(const void* dh, const void* gu, void* dgu, int rows, int inter,
                              cudaStream_t s);
cudaError_t launch_ce_fwd(const void* logits, int64_t ld, const int64_t* labels, float* lse,
                          float* loss_rows, int rows, int vocab, cudaStream_t s);
cudaError_t launch_ce_bwd(void* logits, int64_t ld, const int64_t* labels, const float* lse,
                          const float* scale, int rows, int vocab, cudaStream_t s);
cudaError_t launch_sum_f32(const float* x, float* out, int n, bool accumulate, cudaStream_t s);
cudaError_t launch_embedding_scatter_add(const float* dx, const int64_t* ids, float* dw, int rows,
                                         int cols, int64_t vocab, int64_t pad_id, cudaStream_t s);
cudaError_t launch_cast_f32_to_bf16(const float* x, void* y, int64_t n, cudaStream_t s);
cudaError_t launch_add_f32(const float* a, const float* b, float* out, int64_t n, cudaStream_t s);

// Optimiser over a flat fp32 arena (one launch for every shard leaf).
struct AdamWArgs {
  float lr, beta1, beta2, eps, weight_decay;
  float bias_correction1, bias_correction2;  // 1 - beta^t
  float grad_scale;                          // multiplies the gradient first (1/F etc.)
};
cudaError_t launch_adamw(float* p, const float* g, float* m, float* v, int64_t n, AdamWArgs a,
                         cudaStream_t s);
cudaError_t launch_sgd(float* p, const float* g, int64_t n, float lr, cudaStream_t s);
// flags[0] |= any non-finite in g[0,n) ; flags[1] |= any non-zero in the listed padding ranges.
cudaError_t launch_grad_check(const float* g, int64_t n, const int64_t* pad_ranges, int n_ranges,
                              int* flags, cudaStream_t s);

// Packing for the library-collective (NCCL) path: `table` is an int64 device tensor with one row
// {start in slot, shard length q, numel, offset in the flat output} per parameter of the unit.
// unpack: rank-major gather buffer [degree, slot] -> the unit's parameters, contiguous in `out`.
// pack: full gradients (device array of pointers) -> destination-major [degree, slot], zero padded.
// `largest`: the largest numel (unpack) or shard length q (pack) in the table, for the grid size.
cudaError_t launch_unpack_gathered(const float* packed, int64_t slot, const int64_t* table,
                                   int n_params, int64_t largest, float* out, cudaStream_t s);
cudaError_t launch_pack_gradients(const int64_t* grads, const int64_t* table, int n_params, int degree,
                                  int64_t slot, int64_t used, int64_t largest, float* packed,
                                  cudaStream_t s);

// ------------------------------------------------------------------ shard <-> full (peer.cu)
// One entry per parameter of a unit.  The FSDP shard of parameter j on rank r is elements
// [r*q, min((r+1)*q, numel)) of the TP-local flattened tensor, stored at shard_off in every
// rank's shard arena (zero padded to q).
struct SegmentDesc {
  int64_t shard_off;  // element offset inside the unit's shard arena (same on all ranks)
  int64_t q;          // shard length ceil(numel / F)
  int64_t numel;      // TP-local numel
  int64_t full_off;   // element offset inside the unit's full buffers
  int32_t keep_fp32;  // materialise as fp32 into the small fp32 buffer instead of bf16
  int32_t pad;        // reduce-scatter only: non-zero marks a TP-replicated parameter
};
constexpr int kMaxPeers = 8;
struct PeerPtrs {
  const float* p[kMaxPeers];
};
struct PeerPtrsMut {
  float* p[kMaxPeers];
};
// All-gather fused with the fp32 -> bf16 cast: every rank pulls the peers' fp32 shards over
// NVLink with plain loads and lands the compute-dtype full parameters locally.  With `shadows`
// (one bf16 arena per peer, same element offsets as the fp32 shard arena, kept current by the
// optimizer kernels) the bf16 segments are pulled from there instead: half the bytes on the wire.
cudaError_t launch_gather_params(PeerPtrs shards, int degree, const SegmentDesc* segs, int n_segs,
                                 void* full_bf16, float* full_fp32, int64_t total_full,
                                 cudaStream_t s, const void* const* shadows = nullptr);
// Tensor-parallel axis of a gradient reduction.  With degree > 1 the pointer table lists the
// whole mesh (index f * degree + t); segments whose `pad` field is non-zero are TP-replicated
// parameters, summed over every rank of the mesh and scaled by replicated_scale.
struct TpAxis {
  int degree = 1;
  int rank = 0;
  float replicated_scale = 1.f;
};
// Reduce-scatter fused with the fp32 accumulate into the persistent gradient shard: rank r pulls
// its slice of every peer's full fp32 gradient, sums, scales and adds (or stores).
cudaError_t launch_reduce_scatter_grads(PeerPtrs full_grads, int degree, int rank,
                                        const SegmentDesc* segs, int n_segs, float* grad_shard,
                                        int64_t shard_total, float scale, bool accumulate,
                                        int* flags, cudaStream_t s, TpAxis tp = TpAxis{},
                                        const int* status = nullptr,
                                        const float* multicast = nullptr);
// Same, and applies AdamW to the owned shard in the same pass (last micro-step only).
// `flags` (optional, int[2]) receives the gradient check of what was written: [0] non-finite
// value, [1] non-zero shard padding.
cudaError_t launch_reduce_scatter_adamw(PeerPtrs full_grads, int degree, int rank,
                                        const SegmentDesc* segs, int n_segs, float* grad_shard,
                                        float* p, float* m, float* v, int64_t shard_total,
                                        float scale, bool accumulate, AdamWArgs a, int* flags,
                                        cudaStream_t s, TpAxis tp = TpAxis{},
                                        void* shadow = nullptr,    // bf16 copy of p, same offsets
                                        const int* status = nullptr,
                                        const float* multicast = nullptr);
// `multicast` (both reductions, optional): NVLS multicast address of the gradient slots whose
// unicast addresses `full_grads` lists (memory bound to an NVLink multicast object spanning
// exactly the `degree` FSDP members).  TP-split parameters are then summed by the switch
// (`multimem.ld_reduce`, 16 bytes at a time); TP-replicated parameters, unaligned tails and
// everything else keep the fixed-order peer loads.
// `status` (both reductions): when the word already holds a failure code on entry the kernel
// returns without touching gradients or parameters (the data it would reduce may be stale).
// ------------------------------------------------------------------ all-gather -> GEMM (gemm_allgather_sm100.cu)
// One FSDP-sharded parameter of the fused weight: `rows` consecutive rows of W, stored flat
// ([rows * K] elements) and cut into F shards of q elements that sit at `shard_off` in every
// rank's arena; `full_off` is where the parameter starts in the local full (gathered) buffer.
struct AgSegment {
  int64_t shard_off, q, full_off;
  int rows;
};
struct AgWeights {
  const __nv_bfloat16* shadow[kMaxPeers];  // bf16 arenas (one per FSDP rank); shadow[0] == nullptr
  const float* shard[kMaxPeers];           // ... selects the fp32 arenas (fp32 on the wire)
  int degree;
  int n_segs;                              // 1..4 parameters, in row order of the fused weight
  AgSegment seg[4];
  __nv_bfloat16* full;                     // optional: the pulled rows are also stored here
};
// out[M, N] = a[M, K] * W[N, K]^T (+ bias), W pulled from the FSDP ranks' arenas inside the GEMM
// (peer pointers are read with plain loads; tensor maps cover local memory only).  Gated mode
// (gated_inter > 0): W = gate|up (two segments of gated_inter rows), out = [M, 2 * gated_inter]
// gate|up and gated_out = [M, gated_inter] silu(gate) * up, all bf16.  When M needs more row
// tiles than TMEM holds accumulators (512 / tile width), `w.full` is required: later passes read
// the weight from there instead of crossing the link again.
struct AgGemmCall {
  const void* a;        // bf16 [M, lda], local
  void* out;            // bf16 [M, ldo]
  const float* bias;    // optional fp32 [N]
  void* gated_out;
  int M, N, K;
  int64_t lda, ldo;
  int gated_inter;
  int force_bn;         // 0 = rule, else 64 or 128 (plain mode only)
  AgWeights w;
};
cudaError_t launch_gemm_allgather(const AgGemmCall& c, int* status, cudaStream_t stream);

// Embedding lookup straight from the (possibly remote) fp32 shards: no all-gather of the table.
cudaError_t launch_embedding_gather_sharded(PeerPtrs shards, int degree, int64_t q,
                                            const int64_t* ids, float* out, int rows, int cols,
                                            cudaStream_t s);
// Sequence all-gather of an activation: out[b, r*sl + s, :] = peer r's x[b, s, :].
cudaError_t launch_seq_gather(const void* const* peers, int degree, void* out, int batch,
                              int seq_local, int64_t row_bytes, cudaStream_t s);
// Sequence reduce-scatter: out[b, s, :] = sum_r peer r's partial[b, rank*sl + s, :] (+ residual).
cudaError_t launch_seq_reduce_scatter_f32(const float* const* peers, int degree, int rank,
                                          const float* residual, float* out, int batch,
                                          int seq_local, int cols, cudaStream_t s);
// Cross-GPU barrier over flag words in peer memory.  The wait is bounded by `budget_ns`
// nanoseconds of the global timer; on expiry the status block records {code, silent member,
// epoch awaited, epoch seen}.  With a failure already recorded the kernel publishes its epoch
// and returns without waiting.
cudaError_t launch_peer_barrier(uint32_t* const* flag_pads, int degree, int rank, uint32_t epoch,
                                int slot, int* status, uint64_t budget_ns, cudaStream_t s);

// All-reduce of up to 16 doubles over peer memory in one launch (the per-step metrics: valid-label
// count, loss numerator, finite vote).  Element i is summed, or minimised when bit i of min_mask
// is set; every rank combines the contributions in rank order.  inboxes[r]: rank r's
// [2][8][16]-double inbox.  Bounded wait, status word on expiry.
cudaError_t launch_peer_allreduce_small(uint32_t* const* flag_pads, double* const* inboxes, int degree,
                                        int rank, uint32_t epoch, int slot, const double* in,
                                        double* out, int n, uint32_t min_mask, int* status,
                                        uint64_t budget_ns, cudaStream_t s);

// ------------------------------------------------------------------ attention (attention_sm100.cu)
struct AttnCall {
  const void* qkv;   // bf16 [B*S, (hq + 2 hkv) * 128], rope already applied
  void* out;         // bf16 [B*S, hq*128]
  float* lse;        // fp32 [B, hq, S]
  const uint8_t* key_mask;  // optional [B, S] (1 = attend)
  int batch, seq, hq, hkv;
  float scale;
  // Optional packed form of the key mask (takes precedence over key_mask): bit i of word w of
  // sample b is key 32 w + i; `key_bits_pitch` words per sample (a multiple of 4, at least four
  // per 128-key block; 16-byte aligned).  Written by launch_pack_key_mask, once per batch
  // instead of one byte load per key, block and query row.
  const uint32_t* key_bits;
  int key_bits_pitch;
};
cudaError_t launch_pack_key_mask(const uint8_t* mask, uint32_t* bits, int batch, int seq, int pitch,
                                 cudaStream_t s);
cudaError_t launch_attention_fwd(const AttnCall& c, int* status, cudaStream_t s);
struct AttnBwdCall {
  const void* qkv;
  const void* out;
  const void* dout;  // bf16 [B*S, hq*128]
  const float* lse;
  float* delta;      // fp32 [B, hq, S] scratch
  void* dqkv;        // bf16 [B*S, (hq + 2 hkv) * 128]
  // Optional fp32 scratch of attention_bwd_parts(...) * B*S * 2*hkv*128 floats.  When given, the
  // query heads of a GQA group are split over that many dK/dV CTAs per kv head (small batches
  // would otherwise occupy few SMs) and the partial planes are added in a fixed order.
  float* dkv_accum;
  int64_t dkv_accum_floats;
  const uint8_t* key_mask;
  int batch, seq, hq, hkv;
  float scale;
  const uint32_t* key_bits;   // as in AttnCall
  int key_bits_pitch;
};
cudaError_t launch_attention_bwd(const AttnBwdCall& c, int* status, cudaStream_t s);
int attention_bwd_parts(int batch, int seq, int hq, int hkv);

}  // namespace stb
