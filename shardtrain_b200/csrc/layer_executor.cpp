// Native executor of one Qwen2 decoder layer: the whole forward (10 or 11 launches) or backward
// (26 launches) sequence is issued from C++ in one call, so the host cost per layer is a few
// microseconds per launch instead of a Python round trip per kernel.  The math and the launch
// order are those documented in shardtrain_b200/runtime/fused.py (FusedLayerFn); this file only
// moves the sequencing off the interpreter.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <torch/library.h>

#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "api.h"

namespace {

using at::Tensor;

void ok(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, "shardtrain_b200 layer executor: ", what, ": ", cudaGetErrorString(e));
}

// The key mask of a layer call: a uint8 [B, S] tensor, or (faster) its packed int32 [B, pitch]
// form with one bit per key (ops.pack_key_mask).
struct MaskView {
  const uint8_t* bytes = nullptr;
  const uint32_t* bits = nullptr;
  int pitch = 0;
  explicit MaskView(const c10::optional<at::Tensor>& mask) {
    if (!mask.has_value()) return;
    if (mask->scalar_type() == at::kInt) {
      TORCH_CHECK(mask->dim() == 2 && mask->is_contiguous(), "packed key mask must be [B, words]");
      bits = reinterpret_cast<const uint32_t*>(mask->data_ptr<int>());
      pitch = static_cast<int>(mask->size(1));
    } else {
      bytes = mask->data_ptr<uint8_t>();
    }
  }
};

// Optional "pull the weights inside the GEMM" plan of a layer forward: the FSDP ranks' arenas
// and, for q|k|v and gate|up, the rows of the unit's gather table that describe those parameters.
// Empty `arenas`: the weights were gathered beforehand and the plain GEMMs run.
struct AgPlan {
  std::vector<int64_t> arenas;
  bool wire_fp32 = false;
  const at::Tensor* segs_qkv = nullptr;   // CPU int64 [3, 5]
  const at::Tensor* segs_gu = nullptr;    // CPU int64 [2, 5]
  at::Tensor full;                        // the unit's local bf16 full-parameter buffer
  bool on() const { return !arenas.empty(); }
};

AgPlan make_ag_plan(c10::ArrayRef<int64_t> arenas, bool wire_fp32,
                    const c10::optional<at::Tensor>& segs_qkv,
                    const c10::optional<at::Tensor>& segs_gu,
                    const c10::optional<at::Tensor>& full) {
  AgPlan plan;
  if (arenas.empty()) return plan;
  TORCH_CHECK((segs_qkv.has_value() || segs_gu.has_value()) && full.has_value(),
              "fused all-gather: a segment table and the full buffer are required");
  plan.arenas.assign(arenas.begin(), arenas.end());
  plan.wire_fp32 = wire_fp32;
  plan.segs_qkv = segs_qkv.has_value() ? &*segs_qkv : nullptr;     // either may stay with the
  plan.segs_gu = segs_gu.has_value() ? &*segs_gu : nullptr;        // gather kernel
  plan.full = *full;
  return plan;
}

// Sequence all-gather of a GEMM's A operand inside the GEMM: the peers' [B * Sl, K] slices.
struct SeqPull {
  c10::ArrayRef<int64_t> peers;
  int64_t batch = 0, seq_local = 0;
  bool on() const { return peers.size() > 1; }
};

struct Gemm {
  cudaStream_t stream;
  int* status;
  static void set_pull(stb::GemmCall& c, const SeqPull& pull, int64_t src_ld) {
    if (!pull.on()) return;
    c.pull_degree = static_cast<int>(pull.peers.size());
    c.pull_batch = static_cast<int>(pull.batch);
    c.pull_seq_local = static_cast<int>(pull.seq_local);
    c.pull_src_ld = src_ld;
    for (size_t i = 0; i < pull.peers.size(); ++i)
      c.pull_peers[i] = reinterpret_cast<const void*>(pull.peers[i]);
  }
  // out = a @ W^T (+ bias) [+ SwiGLU into hm] with W pulled from the FSDP ranks inside the GEMM
  void allgather(const Tensor& a, Tensor& out, const float* bias, Tensor* hm, const AgPlan& plan,
                 const at::Tensor& segs) const {
    TORCH_CHECK(!segs.is_cuda() && segs.scalar_type() == at::kLong && segs.dim() == 2 &&
                    segs.size(1) == 5 && segs.size(0) >= 1 && segs.size(0) <= 4 &&
                    segs.is_contiguous(), "fused all-gather: bad segment table");
    stb::AgGemmCall c{};
    c.a = a.data_ptr();
    c.out = out.data_ptr();
    c.bias = bias;
    c.M = static_cast<int>(a.size(0));
    c.K = static_cast<int>(a.size(1));
    c.N = static_cast<int>(out.size(1));
    c.lda = a.stride(0);
    c.ldo = out.stride(0);
    if (hm != nullptr) {
      c.gated_out = hm->data_ptr();
      c.gated_inter = static_cast<int>(hm->size(1));
    }
    c.w.degree = static_cast<int>(plan.arenas.size());
    for (size_t i = 0; i < plan.arenas.size(); ++i) {
      if (plan.wire_fp32)
        c.w.shard[i] = reinterpret_cast<const float*>(plan.arenas[i]);
      else
        c.w.shadow[i] = reinterpret_cast<const __nv_bfloat16*>(plan.arenas[i]);
    }
    const int64_t* t = segs.data_ptr<int64_t>();
    c.w.n_segs = static_cast<int>(segs.size(0));
    for (int j = 0; j < c.w.n_segs; ++j) {
      c.w.seg[j].shard_off = t[5 * j];
      c.w.seg[j].q = t[5 * j + 1];
      TORCH_CHECK(t[5 * j + 2] % c.K == 0, "fused all-gather: a parameter is not whole rows");
      c.w.seg[j].rows = static_cast<int>(t[5 * j + 2] / c.K);
      c.w.seg[j].full_off = t[5 * j + 3];
    }
    c.w.full = reinterpret_cast<__nv_bfloat16*>(plan.full.data_ptr());
    ok(stb::launch_gemm_allgather(c, status, stream), "gemm all-gather");
  }
  // `pull`: `a` is the local buffer that the GEMM first fills from the peers' sequence slices
  void run(const Tensor& a, const Tensor& b, Tensor& out, bool a_mn, bool b_mn, const float* bias,
           const Tensor* residual, const SeqPull& pull = SeqPull{}) const {
    stb::GemmCall c{};
    set_pull(c, pull, a.stride(0));
    c.M = static_cast<int>(a_mn ? a.size(1) : a.size(0));
    c.K = static_cast<int>(a_mn ? a.size(0) : a.size(1));
    c.N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
    c.a = a.data_ptr();
    c.b = b.data_ptr();
    c.out = out.data_ptr();
    c.lda = a.stride(0);
    c.ldb = b.stride(0);
    c.ldo = out.stride(0);
    c.a_mn = a_mn;
    c.b_mn = b_mn;
    c.out_fp32 = out.scalar_type() == at::kFloat;
    c.accumulate = false;
    c.alpha = 1.f;
    c.force_bn = 0;
    c.bias = bias;
    c.residual = residual ? residual->data_ptr() : nullptr;
    ok(stb::launch_gemm_bf16(c, status, stream), "gemm");
  }
  // gate|up projection with the SwiGLU epilogue: gu = a @ w_gu^T, hm = silu(gate) * up
  void swiglu(const Tensor& a, const Tensor& w_gu, Tensor& gu, Tensor& hm,
              const SeqPull& pull = SeqPull{}) const {
    stb::GemmCall c{};
    set_pull(c, pull, a.stride(0));
    c.M = static_cast<int>(a.size(0));
    c.K = static_cast<int>(a.size(1));
    c.N = static_cast<int>(w_gu.size(0));
    c.a = a.data_ptr();
    c.b = w_gu.data_ptr();
    c.out = gu.data_ptr();
    c.lda = a.stride(0);
    c.ldb = w_gu.stride(0);
    c.ldo = gu.stride(0);
    c.alpha = 1.f;
    c.gated_out = hm.data_ptr();
    c.gated_inter = static_cast<int>(hm.size(1));
    ok(stb::launch_gemm_bf16(c, status, stream), "gemm swiglu");
  }
  // q|k|v projection (+ bias), pulling the weights inside the GEMM when a plan is given
  void qkv_proj(const Tensor& a, const Tensor& w_qkv, Tensor& qkv, const float* bias,
                const AgPlan& plan, const SeqPull& pull = SeqPull{}) const {
    if (plan.on() && plan.segs_qkv != nullptr)
      allgather(a, qkv, bias, nullptr, plan, *plan.segs_qkv);
    else
      run(a, w_qkv, qkv, false, false, bias, nullptr, pull);
  }
  // fp32 partial rows pushed into every TP rank's receive slot (all-reduce without SP)
  void broadcast(const Tensor& a, const Tensor& b, bool b_mn, c10::ArrayRef<int64_t> dest) const {
    stb::GemmCall c{};
    c.M = static_cast<int>(a.size(0));
    c.K = static_cast<int>(a.size(1));
    c.N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
    c.a = a.data_ptr();
    c.b = b.data_ptr();
    c.lda = a.stride(0);
    c.ldb = b.stride(0);
    c.ldo = c.N;
    c.b_mn = b_mn;
    c.out_fp32 = true;
    c.alpha = 1.f;
    c.scatter_degree = static_cast<int>(dest.size());
    c.scatter_broadcast = 1;
    for (size_t i = 0; i < dest.size(); ++i) c.scatter_out[i] = reinterpret_cast<float*>(dest[i]);
    c.out = c.scatter_out[0];
    ok(stb::launch_gemm_bf16(c, status, stream), "gemm broadcast");
  }
  // gate|up projection with SwiGLU in the GEMM epilogue (the epilogue leaves through staged TMA
  // stores).  Measured on B200 against GEMM + SwiGLU kernel, bit-identical results: 40 us against
  // 47 us at 512 rows, 61 / 69 at 1024, 103 / 114 at 2048, 187 / 210 at 4096.
  void gate_up(const Tensor& a, const Tensor& w_gu, Tensor& gu, Tensor& hm, cudaStream_t,
               const AgPlan& plan = AgPlan{}, const SeqPull& pull = SeqPull{}) const {
    if (plan.on() && plan.segs_gu != nullptr) {
      allgather(a, gu, nullptr, &hm, plan, *plan.segs_gu);
      return;
    }
    swiglu(a, w_gu, gu, hm, pull);
  }
  // fp32 result rows scattered along the sequence into the owners' receive slots (peer memory)
  void scatter(const Tensor& a, const Tensor& b, bool b_mn, c10::ArrayRef<int64_t> dest, int seq) const {
    stb::GemmCall c{};
    c.M = static_cast<int>(a.size(0));
    c.K = static_cast<int>(a.size(1));
    c.N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
    c.a = a.data_ptr();
    c.b = b.data_ptr();
    c.lda = a.stride(0);
    c.ldb = b.stride(0);
    c.ldo = c.N;
    c.b_mn = b_mn;
    c.out_fp32 = true;
    c.alpha = 1.f;
    c.scatter_degree = static_cast<int>(dest.size());
    c.scatter_seq = seq;
    c.scatter_seq_local = seq / static_cast<int>(dest.size());
    for (size_t i = 0; i < dest.size(); ++i) c.scatter_out[i] = reinterpret_cast<float*>(dest[i]);
    c.out = c.scatter_out[0];
    ok(stb::launch_gemm_bf16(c, status, stream), "gemm scatter");
  }
};

// Sequence-parallel plumbing of one layer call: the TP group's flag pads for the in-stream
// barrier, and the epoch counter the caller advances by the number of barriers used.
struct SpLink {
  cudaStream_t stream;
  int* status;
  std::vector<uint32_t*> pads;
  int rank;
  uint32_t epoch;
  int slot;
  uint64_t budget_ns;
  void barrier() {
    ++epoch;
    ok(stb::launch_peer_barrier(pads.data(), static_cast<int>(pads.size()), rank, epoch, slot, status,
                                budget_ns, stream), "sp barrier");
  }
  // out[b, r*sl + s, :] = peer r's [b, s, :]
  void gather(c10::ArrayRef<int64_t> src, Tensor& out, int64_t B, int64_t seq_local) const {
    std::vector<const void*> p(src.size());
    for (size_t i = 0; i < src.size(); ++i) p[i] = reinterpret_cast<const void*>(src[i]);
    ok(stb::launch_seq_gather(p.data(), static_cast<int>(p.size()), out.data_ptr(),
                              static_cast<int>(B), static_cast<int>(seq_local),
                              out.size(1) * out.element_size(), stream), "seq gather");
  }
};

SpLink make_link(cudaStream_t st, int* status, c10::ArrayRef<int64_t> pads, int64_t rank,
                 int64_t epoch, int64_t slot, int64_t wait_us) {
  TORCH_CHECK(wait_us > 0, "the wait budget must be positive (microseconds)");
  SpLink l{st, status, {}, static_cast<int>(rank), static_cast<uint32_t>(epoch),
           static_cast<int>(slot), static_cast<uint64_t>(wait_us) * 1000ull};
  for (int64_t p : pads) l.pads.push_back(reinterpret_cast<uint32_t*>(p));
  return l;
}

// ---------------------------------------------------------------------------------------------
// Replay of launch sequences (CUDA graphs).
//
// A training step presents every decoder layer with the same addresses, shapes and scalars as the
// step before: the weights live in per-unit buffers allocated once, the gradient slots rotate with
// a period that divides the step, and the activations a layer produces are owned here, so they
// too keep their addresses.  A sequence is therefore keyed by EVERYTHING its kernels receive
// (every pointer, pitch and scalar, the stream); the first time a key is seen the sequence is
// launched kernel by kernel into buffers that the cache entry owns, the second time it is
// captured into a graph, and from then on one cudaGraphLaunch replaces the 10 or 26 launches.
// Any difference in the key (another input address, another mask, another shape) is simply a
// different entry; nothing is ever replayed against arguments it was not captured with.
//
// The buffers an entry returns are the SAME tensors at every call.  That is sound for the
// training loop's order -- a layer's forward, then its backward, then the next micro-step's
// forward -- and the Python side asks for a replay only in that order (a second forward of a
// layer before its backward is launched without the cache, into fresh tensors).
struct ReplayEntry {
  std::vector<int64_t> key;
  std::vector<Tensor> buffers;
  cudaGraphExec_t exec = nullptr;
  bool refuse = false;        // capture failed once: this key always launches kernel by kernel
  int64_t kernels = 0;        // launches inside the graph (for the launch counter)
  uint64_t used = 0;
  int64_t bytes = 0;          // device memory held by `buffers`
};

class ReplayCache {
 public:
  // `alloc()` -> the tensors the sequence writes and returns; `launch(buffers)` issues the kernels.
  template <class Alloc, class Launch>
  std::vector<Tensor> run(std::vector<int64_t> key, cudaStream_t st, Alloc&& alloc, Launch&& launch) {
    std::lock_guard<std::mutex> lock(mu_);
    ReplayEntry* e = find(key);
    if (e == nullptr) {
      // Entries keep their buffers: a workload whose keys never repeat (ever-changing shapes or
      // input addresses) must not pile them up.  Past the budget the older half is dropped.
      if (entries_ >= kMaxEntries || bytes_ > budget()) evict();
      e = insert(std::move(key));
      e->buffers = alloc();
      for (const Tensor& b : e->buffers) e->bytes += static_cast<int64_t>(b.nbytes());
      bytes_ += e->bytes;
      launch(e->buffers);
      return e->buffers;
    }
    e->used = ++tick_;
    if (e->exec != nullptr) {
      ok(cudaGraphLaunch(e->exec, st), "graph launch");
      stb::count_launches(e->kernels);
      return e->buffers;
    }
    if (!e->refuse) capture(e, st, launch);
    if (e->exec != nullptr) {
      ok(cudaGraphLaunch(e->exec, st), "graph launch");
    } else {
      e->refuse = true;
      launch(e->buffers);
    }
    return e->buffers;
  }
  size_t graphs() {
    std::lock_guard<std::mutex> lock(mu_);
    size_t n = 0;
    for (auto& kv : table_)
      for (auto& e : kv.second) n += e->exec != nullptr;
    return n;
  }
  void clear() {
    std::lock_guard<std::mutex> lock(mu_);
    for (auto& kv : table_)
      for (auto& e : kv.second)
        if (e->exec != nullptr) cudaGraphExecDestroy(e->exec);
    table_.clear();
    entries_ = 0;
    bytes_ = 0;
  }

 private:
  static uint64_t hash(const std::vector<int64_t>& key) {
    uint64_t h = 0x9e3779b97f4a7c15ull;
    for (int64_t x : key) h = (h ^ static_cast<uint64_t>(x)) * 0x100000001b3ull + (h >> 31);
    return h;
  }
  ReplayEntry* find(const std::vector<int64_t>& key) {
    auto it = table_.find(hash(key));
    if (it == table_.end()) return nullptr;
    for (auto& e : it->second)
      if (e->key == key) return e.get();
    return nullptr;
  }
  // a quarter of the device's memory may sit in replay buffers
  static int64_t budget() {
    static const int64_t value = [] {
      size_t free_bytes = 0, total = 0;
      if (cudaMemGetInfo(&free_bytes, &total) != cudaSuccess) total = size_t{16} << 30;
      return static_cast<int64_t>(total / 4);
    }();
    return value;
  }
  ReplayEntry* insert(std::vector<int64_t> key) {
    auto e = std::make_unique<ReplayEntry>();
    e->key = std::move(key);
    e->used = ++tick_;
    ReplayEntry* raw = e.get();
    table_[hash(raw->key)].push_back(std::move(e));
    ++entries_;
    return raw;
  }
  // Drop the least recently used half (keys that stopped coming back, e.g. after a shape change).
  void evict() {
    std::vector<uint64_t> ages;
    for (auto& kv : table_)
      for (auto& e : kv.second) ages.push_back(e->used);
    if (ages.empty()) return;
    std::nth_element(ages.begin(), ages.begin() + ages.size() / 2, ages.end());
    const uint64_t cut = ages[ages.size() / 2];
    for (auto it = table_.begin(); it != table_.end();) {
      auto& v = it->second;
      for (size_t i = 0; i < v.size();) {
        if (v[i]->used < cut) {
          if (v[i]->exec != nullptr) cudaGraphExecDestroy(v[i]->exec);
          bytes_ -= v[i]->bytes;
          v.erase(v.begin() + i);
          --entries_;
        } else {
          ++i;
        }
      }
      it = v.empty() ? table_.erase(it) : std::next(it);
    }
  }
  template <class Launch>
  void capture(ReplayEntry* e, cudaStream_t st, Launch&& launch) {
    const int64_t before = stb::launches_total();
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
      cudaGetLastError();
      return;
    }
    bool threw = false;
    try {
      launch(e->buffers);
    } catch (...) {
      threw = true;           // the kernel-by-kernel launch that follows reports the error
    }
    cudaGraph_t graph = nullptr;
    const cudaError_t ended = cudaStreamEndCapture(st, &graph);
    if (!threw && ended == cudaSuccess && graph != nullptr) {
      if (cudaGraphInstantiate(&e->exec, graph, 0) != cudaSuccess) e->exec = nullptr;
    }
    if (graph != nullptr) cudaGraphDestroy(graph);
    if (e->exec == nullptr) cudaGetLastError();
    e->kernels = stb::launches_total() - before;
  }

  static constexpr size_t kMaxEntries = 1024;
  std::mutex mu_;
  std::unordered_map<uint64_t, std::vector<std::unique_ptr<ReplayEntry>>> table_;
  size_t entries_ = 0;
  int64_t bytes_ = 0;
  uint64_t tick_ = 0;
};

ReplayCache& replay_cache() {
  static ReplayCache cache;
  return cache;
}

struct KeyBuilder {
  std::vector<int64_t> v;
  KeyBuilder& tag(int64_t t) { v.push_back(t); return *this; }
  KeyBuilder& i(int64_t x) { v.push_back(x); return *this; }
  KeyBuilder& t(const Tensor& x) {
    v.push_back(static_cast<int64_t>(reinterpret_cast<uintptr_t>(x.data_ptr())));
    v.push_back(x.dim() > 0 ? x.size(0) : 1);
    v.push_back(x.dim() > 1 ? x.stride(0) : 1);
    v.push_back(static_cast<int64_t>(x.scalar_type()));
    return *this;
  }
  KeyBuilder& t(const c10::optional<Tensor>& x) {
    if (x.has_value()) return t(*x);
    v.push_back(0);
    return *this;
  }
  KeyBuilder& list(c10::ArrayRef<int64_t> xs) {
    v.push_back(static_cast<int64_t>(xs.size()));
    for (int64_t x : xs) v.push_back(x);
    return *this;
  }
};

// x2 [M,H] fp32 -> {h1, inv1, qkv, attn, lse, x_mid, h2, inv2, gu, out, hm}; hm = silu(gate) * up
// is kept for the backward (73 MB per layer at the headline shape) instead of being recomputed.
// `replay`: serve the call from the replay cache (see above).
std::vector<Tensor> layer_forward(const Tensor& x2, const Tensor& w_qkv, const Tensor& b_qkv,
                                  const Tensor& w_o, const Tensor& w_gu, const Tensor& w_down,
                                  const Tensor& ln1, const Tensor& ln2, const Tensor& cos,
                                  const Tensor& sin, const c10::optional<Tensor>& positions,
                                  const c10::optional<Tensor>& mask, Tensor status, int64_t B,
                                  int64_t S, int64_t hq, int64_t hkv, double eps, c10::ArrayRef<int64_t> ag_arenas,
    bool ag_wire_fp32, const c10::optional<Tensor>& ag_segs_qkv,
    const c10::optional<Tensor>& ag_segs_gu, const c10::optional<Tensor>& ag_full, bool replay) {
  const AgPlan ag = make_ag_plan(ag_arenas, ag_wire_fp32, ag_segs_qkv, ag_segs_gu, ag_full);
  const int64_t M = B * S, H = x2.size(1), D = 128;
  const int64_t W = (hq + 2 * hkv) * D, inter = w_down.size(1);
  auto bf = x2.options().dtype(at::kBFloat16);
  auto f32 = x2.options().dtype(at::kFloat);
  cudaStream_t st = at::cuda::getCurrentCUDAStream().stream();
  Gemm g{st, status.data_ptr<int>()};
  const int* pos = positions.has_value() ? positions->data_ptr<int>() : nullptr;
  const MaskView mv(mask);
  const uint8_t* km = mv.bytes;

  // {h1, inv1, qkv, attn, lse, x_mid, h2, inv2, gu, out, hm}
  auto alloc = [&]() -> std::vector<Tensor> {
    return {at::empty({M, H}, bf),      at::empty({M}, f32),          at::empty({M, W}, bf),
            at::empty({M, hq * D}, bf), at::empty({B, hq, S}, f32),   at::empty({M, H}, f32),
            at::empty({M, H}, bf),      at::empty({M}, f32),          at::empty({M, 2 * inter}, bf),
            at::empty({M, H}, f32),     at::empty({M, inter}, bf)};
  };
  auto launch = [&](std::vector<Tensor>& b) {
    Tensor &h1 = b[0], &inv1 = b[1], &qkv = b[2], &attn = b[3], &lse = b[4], &x_mid = b[5];
    Tensor &h2 = b[6], &inv2 = b[7], &gu = b[8], &out = b[9], &hm = b[10];
    ok(stb::launch_rmsnorm_fwd(x2.data_ptr<float>(), ln1.data_ptr<float>(), h1.data_ptr(),
                               inv1.data_ptr<float>(), M, H, static_cast<float>(eps), false, st), "rmsnorm");
    g.qkv_proj(h1, w_qkv, qkv, b_qkv.data_ptr<float>(), ag);
    ok(stb::launch_rope(qkv.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), pos, M, S, hq,
                        hkv, D, false, st), "rope");
    stb::AttnCall ac{qkv.data_ptr(), attn.data_ptr(), lse.data_ptr<float>(), km, static_cast<int>(B),
                     static_cast<int>(S), static_cast<int>(hq), static_cast<int>(hkv),
                     static_cast<float>(1.0 / std::sqrt(static_cast<double>(D)))};
    ac.key_bits = mv.bits;
    ac.key_bits_pitch = mv.pitch;
    ok(stb::launch_attention_fwd(ac, g.status, st), "attention_fwd");
    g.run(attn, w_o, x_mid, false, false, nullptr, &x2);
    ok(stb::launch_rmsnorm_fwd(x_mid.data_ptr<float>(), ln2.data_ptr<float>(), h2.data_ptr(),
                               inv2.data_ptr<float>(), M, H, static_cast<float>(eps), false, st), "rmsnorm");
    g.gate_up(h2, w_gu, gu, hm, st, ag);
    g.run(hm, w_down, out, false, false, nullptr, &x_mid);
  };
  if (!replay) {
    std::vector<Tensor> b = alloc();
    launch(b);
    return b;
  }
  KeyBuilder k;
  k.tag(1).t(x2).t(w_qkv).t(b_qkv).t(w_o).t(w_gu).t(w_down).t(ln1).t(ln2).t(cos).t(sin).t(positions)
      .t(mask).t(status).i(B).i(S).i(hq).i(hkv).i(H).i(inter);
  int64_t eps_bits = 0;
  static_assert(sizeof(eps_bits) == sizeof(eps), "double is 64 bits");
  std::memcpy(&eps_bits, &eps, sizeof(eps));
  k.i(eps_bits).list(ag_arenas).i(ag_wire_fp32).t(ag_segs_qkv).t(ag_segs_gu).t(ag_full)
      .i(static_cast<int64_t>(reinterpret_cast<uintptr_t>(st)));
  return replay_cache().run(std::move(k.v), st, alloc, launch);
}

// Temporaries of one layer backward.  With replay they are shared by every layer of the same
// shape on the same stream (the layers' backward sequences run one after another on it).
struct BackwardScratch {
  Tensor d_out_b, d_hm, d_gu, d_h2, d_mid, partial, d_mid_b, d_attn, d_qkv, delta, dkv_parts,
      bias_partial, d_h1;
};

constexpr int kNormPartialRows = 592;

BackwardScratch make_backward_scratch(const Tensor& like, int64_t B, int64_t S, int64_t H, int64_t W,
                                      int64_t inter, int64_t hq, int64_t hkv, int parts) {
  const int64_t M = B * S, D = 128;
  auto bf = like.options().dtype(at::kBFloat16);
  auto f32 = like.options().dtype(at::kFloat);
  BackwardScratch s;
  s.d_out_b = at::empty({M, H}, bf);
  s.d_hm = at::empty({M, inter}, bf);
  s.d_gu = at::empty({M, 2 * inter}, bf);
  s.d_h2 = at::empty({M, H}, f32);
  s.d_mid = at::empty({M, H}, f32);
  s.partial = at::empty({kNormPartialRows, H}, f32);
  s.d_mid_b = at::empty({M, H}, bf);
  s.d_attn = at::empty({M, hq * D}, bf);
  s.d_qkv = at::empty({M, W}, bf);
  s.delta = at::empty({B, hq, S}, f32);
  if (parts > 1) s.dkv_parts = at::empty({parts, M, 2 * hkv * D}, f32);
  s.bias_partial = at::empty({64, W}, f32);
  s.d_h1 = at::empty({M, H}, f32);
  return s;
}

BackwardScratch& shared_backward_scratch(const Tensor& like, int64_t B, int64_t S, int64_t H,
                                         int64_t W, int64_t inter, int64_t hq, int64_t hkv,
                                         int parts, cudaStream_t st) {
  static std::mutex mu;
  static std::map<std::vector<int64_t>, BackwardScratch> table;
  std::vector<int64_t> key{like.get_device(), B, S, H, W, inter, hq, hkv, parts,
                           static_cast<int64_t>(reinterpret_cast<uintptr_t>(st))};
  std::lock_guard<std::mutex> lock(mu);
  auto it = table.find(key);
  if (it == table.end())
    it = table.emplace(key, make_backward_scratch(like, B, S, H, W, inter, hq, hkv, parts)).first;
  return it->second;
}

// Gradient views (down, gate_up, ln2, o, bias, qkv, ln1) point into the unit's gradient slot.
Tensor layer_backward(const Tensor& d_out, const Tensor& x2, const Tensor& inv1, const Tensor& h1,
                      const Tensor& qkv, const Tensor& attn, const Tensor& lse, const Tensor& x_mid,
                      const Tensor& inv2, const Tensor& h2, const Tensor& gu, const Tensor& hm,
                      const Tensor& w_qkv,
                      const Tensor& w_o, const Tensor& w_gu, const Tensor& w_down, const Tensor& ln1,
                      const Tensor& ln2, Tensor g_down, Tensor g_gate_up, Tensor g_ln2, Tensor g_o,
                      Tensor g_bias, Tensor g_qkv, Tensor g_ln1, const Tensor& cos, const Tensor& sin,
                      const c10::optional<Tensor>& positions, const c10::optional<Tensor>& mask,
                      Tensor status, int64_t B, int64_t S, int64_t hq, int64_t hkv, bool replay) {
  const int64_t M = B * S, H = x2.size(1), D = 128;
  const int64_t W = (hq + 2 * hkv) * D, inter = w_down.size(1);
  auto f32 = x2.options().dtype(at::kFloat);
  cudaStream_t st = at::cuda::getCurrentCUDAStream().stream();
  Gemm g{st, status.data_ptr<int>()};
  const int* pos = positions.has_value() ? positions->data_ptr<int>() : nullptr;
  const MaskView mv(mask);
  const uint8_t* km = mv.bytes;
  const int parts = stb::attention_bwd_parts(static_cast<int>(B), static_cast<int>(S),
                                             static_cast<int>(hq), static_cast<int>(hkv));
  BackwardScratch own;
  if (!replay) own = make_backward_scratch(x2, B, S, H, W, inter, hq, hkv, parts);
  BackwardScratch& t = replay ? shared_backward_scratch(x2, B, S, H, W, inter, hq, hkv, parts, st) : own;

  auto alloc = [&]() -> std::vector<Tensor> { return {at::empty({M, H}, f32)}; };
  auto launch = [&](std::vector<Tensor>& b) {
    Tensor& dx = b[0];
    ok(stb::launch_cast_f32_to_bf16(d_out.data_ptr<float>(), t.d_out_b.data_ptr(), M * H, st), "cast");
    g.run(t.d_out_b, hm, g_down, true, true, nullptr, nullptr);                 // dW down
    g.run(t.d_out_b, w_down, t.d_hm, false, true, nullptr, nullptr);            // dX down
    ok(stb::launch_swiglu_bwd(t.d_hm.data_ptr(), gu.data_ptr(), t.d_gu.data_ptr(), M, inter, st), "swiglu_bwd");
    g.run(t.d_gu, h2, g_gate_up, true, true, nullptr, nullptr);                 // dW gate|up
    g.run(t.d_gu, w_gu, t.d_h2, false, true, nullptr, nullptr);                 // dX gate|up
    ok(stb::launch_rmsnorm_bwd(t.d_h2.data_ptr<float>(), x_mid.data_ptr<float>(), ln2.data_ptr<float>(),
                               inv2.data_ptr<float>(), d_out.data_ptr<float>(), t.d_mid.data_ptr<float>(),
                               t.partial.data_ptr<float>(), kNormPartialRows, M, H, st), "rmsnorm_bwd");
    ok(stb::launch_colsum_f32(t.partial.data_ptr<float>(), g_ln2.data_ptr<float>(), kNormPartialRows, H,
                              false, st), "colsum");
    ok(stb::launch_cast_f32_to_bf16(t.d_mid.data_ptr<float>(), t.d_mid_b.data_ptr(), M * H, st), "cast");
    g.run(t.d_mid_b, attn, g_o, true, true, nullptr, nullptr);                  // dW o
    g.run(t.d_mid_b, w_o, t.d_attn, false, true, nullptr, nullptr);             // dX o
    stb::AttnBwdCall bc{};
    bc.qkv = qkv.data_ptr();
    bc.out = attn.data_ptr();
    bc.dout = t.d_attn.data_ptr();
    bc.lse = lse.data_ptr<float>();
    bc.delta = t.delta.data_ptr<float>();
    bc.dqkv = t.d_qkv.data_ptr();
    bc.dkv_accum = parts > 1 ? t.dkv_parts.data_ptr<float>() : nullptr;
    bc.dkv_accum_floats = parts > 1 ? t.dkv_parts.numel() : 0;
    bc.key_mask = km;
    bc.key_bits = mv.bits;
    bc.key_bits_pitch = mv.pitch;
    bc.batch = static_cast<int>(B);
    bc.seq = static_cast<int>(S);
    bc.hq = static_cast<int>(hq);
    bc.hkv = static_cast<int>(hkv);
    bc.scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(D)));
    ok(stb::launch_attention_bwd(bc, g.status, st), "attention_bwd");
    ok(stb::launch_rope(t.d_qkv.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), pos, M, S, hq,
                        hkv, D, true, st), "rope inverse");
    ok(stb::launch_colsum_bf16(t.d_qkv.data_ptr(), W, g_bias.data_ptr<float>(), M, W, false,
                               t.bias_partial.data_ptr<float>(), 64, st), "bias colsum");
    g.run(t.d_qkv, h1, g_qkv, true, true, nullptr, nullptr);                    // dW q|k|v
    g.run(t.d_qkv, w_qkv, t.d_h1, false, true, nullptr, nullptr);               // dX q|k|v
    ok(stb::launch_rmsnorm_bwd(t.d_h1.data_ptr<float>(), x2.data_ptr<float>(), ln1.data_ptr<float>(),
                               inv1.data_ptr<float>(), t.d_mid.data_ptr<float>(), dx.data_ptr<float>(),
                               t.partial.data_ptr<float>(), kNormPartialRows, M, H, st), "rmsnorm_bwd");
    ok(stb::launch_colsum_f32(t.partial.data_ptr<float>(), g_ln1.data_ptr<float>(), kNormPartialRows, H,
                              false, st), "colsum");
  };
  if (!replay) {
    std::vector<Tensor> b = alloc();
    launch(b);
    return b[0];
  }
  KeyBuilder k;
  k.tag(2).t(d_out).t(x2).t(inv1).t(h1).t(qkv).t(attn).t(lse).t(x_mid).t(inv2).t(h2).t(gu).t(hm)
      .t(w_qkv).t(w_o).t(w_gu).t(w_down).t(ln1).t(ln2).t(g_down).t(g_gate_up).t(g_ln2).t(g_o)
      .t(g_bias).t(g_qkv).t(g_ln1).t(cos).t(sin).t(positions).t(mask).t(status).i(B).i(S).i(hq)
      .i(hkv).i(H).i(inter).i(static_cast<int64_t>(reinterpret_cast<uintptr_t>(st)));
  return replay_cache().run(std::move(k.v), st, alloc, launch)[0];
}

// ---------------------------------------------------------------------------------------------
// Tensor + sequence parallel layer.  The residual stream is sequence sharded ([B, S/T, H] per TP
// rank); column-parallel GEMMs consume a sequence all-gather of the normalised activations (one
// gather feeds q|k|v, one feeds gate|up -- src/sharded_runtime/runtime/qwen2_operators.py:253-265),
// row-parallel GEMMs scatter their fp32 partial sums from the epilogue straight into the owning
// rank's receive slots over NVLink, and the next kernel adds the T slots (+ residual, + RMSNorm).
// h1 / h2 / bf16 output gradients live in peer-visible buffers so the peers' gathers (and the
// backward's re-gathers) read them in place.
//
// x2 [B*S/T, H] fp32 -> {inv1, qkv, attn, lse, x_mid, inv2, gu, out, hm}; uses 4 barrier epochs.
std::vector<Tensor> layer_forward_sp(
    const Tensor& x2, const Tensor& w_qkv, const Tensor& b_qkv, const Tensor& w_o,
    const Tensor& w_gu, const Tensor& w_down, const Tensor& ln1, const Tensor& ln2,
    const Tensor& cos, const Tensor& sin, const c10::optional<Tensor>& positions,
    const c10::optional<Tensor>& mask, Tensor status, int64_t B, int64_t S, int64_t hq,
    int64_t hkv, double eps, Tensor h1_local, Tensor h2_local, c10::ArrayRef<int64_t> h1_ptrs,
    c10::ArrayRef<int64_t> h2_ptrs, c10::ArrayRef<int64_t> push_ptrs, Tensor recv,
    c10::ArrayRef<int64_t> flag_ptrs, int64_t tp_rank, int64_t epoch, int64_t flag_slot,
    int64_t wait_us, bool seq_pull, c10::ArrayRef<int64_t> ag_arenas,
    bool ag_wire_fp32, const c10::optional<Tensor>& ag_segs_qkv,
    const c10::optional<Tensor>& ag_segs_gu, const c10::optional<Tensor>& ag_full) {
  const AgPlan ag = make_ag_plan(ag_arenas, ag_wire_fp32, ag_segs_qkv, ag_segs_gu, ag_full);
  const int64_t T = static_cast<int64_t>(h1_ptrs.size());
  const int64_t Sl = S / T, Ml = B * Sl, M = B * S, H = x2.size(1), D = 128;
  // the sequence gather runs inside the consuming GEMM unless that GEMM already pulls its weights
  const bool pull_qkv = seq_pull && !(ag.on() && ag.segs_qkv != nullptr);
  const bool pull_gu = seq_pull && !(ag.on() && ag.segs_gu != nullptr);
  const int64_t W = (hq + 2 * hkv) * D, inter = w_down.size(1);
  TORCH_CHECK(S % T == 0 && x2.size(0) == Ml && recv.dim() == 3 && recv.size(0) == T &&
                  recv.size(1) == Ml && recv.size(2) == H && recv.is_contiguous(),
              "sequence-parallel layer: shapes do not match the TP degree");
  auto bf = x2.options().dtype(at::kBFloat16);
  auto f32 = x2.options().dtype(at::kFloat);
  cudaStream_t st = at::cuda::getCurrentCUDAStream().stream();
  Gemm g{st, status.data_ptr<int>()};
  SpLink sp = make_link(st, g.status, flag_ptrs, tp_rank, epoch, flag_slot, wait_us);
  const int* pos = positions.has_value() ? positions->data_ptr<int>() : nullptr;
  const MaskView mv(mask);
  const uint8_t* km = mv.bytes;
  const float feps = static_cast<float>(eps);

  Tensor inv1 = at::empty({Ml}, f32);
  ok(stb::launch_rmsnorm_fwd(x2.data_ptr<float>(), ln1.data_ptr<float>(), h1_local.data_ptr(),
                             inv1.data_ptr<float>(), Ml, H, feps, false, st), "rmsnorm");
  sp.barrier();                                   // every rank's h1 slice is written
  Tensor h_full = at::empty({M, H}, bf);
  if (!pull_qkv) sp.gather(h1_ptrs, h_full, B, Sl);
  Tensor qkv = at::empty({M, W}, bf);
  g.qkv_proj(h_full, w_qkv, qkv, b_qkv.data_ptr<float>(), ag,
             pull_qkv ? SeqPull{h1_ptrs, B, Sl} : SeqPull{});
  ok(stb::launch_rope(qkv.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), pos, M, S, hq,
                      hkv, D, false, st), "rope");
  Tensor attn = at::empty({M, hq * D}, bf), lse = at::empty({B, hq, S}, f32);
  stb::AttnCall ac{qkv.data_ptr(), attn.data_ptr(), lse.data_ptr<float>(), km, static_cast<int>(B),
                   static_cast<int>(S), static_cast<int>(hq), static_cast<int>(hkv),
                   static_cast<float>(1.0 / std::sqrt(static_cast<double>(D)))};
  ac.key_bits = mv.bits;
  ac.key_bits_pitch = mv.pitch;
  ok(stb::launch_attention_fwd(ac, g.status, st), "attention_fwd");
  g.scatter(attn, w_o, false, push_ptrs, static_cast<int>(S));
  sp.barrier();                                   // every rank's partial rows have landed
  Tensor x_mid = at::empty({Ml, H}, f32), inv2 = at::empty({Ml}, f32);
  ok(stb::launch_slot_sum_rmsnorm(recv.data_ptr<float>(), T, recv.stride(0), x2.data_ptr<float>(),
                                  x_mid.data_ptr<float>(), ln2.data_ptr<float>(),
                                  h2_local.data_ptr(), inv2.data_ptr<float>(), Ml, H, feps, st),
     "slot sum + rmsnorm");
  sp.barrier();                                   // h2 slices written, receive slots consumed
  if (!pull_gu) sp.gather(h2_ptrs, h_full, B, Sl);
  Tensor gu = at::empty({M, 2 * inter}, bf), hm = at::empty({M, inter}, bf);
  g.gate_up(h_full, w_gu, gu, hm, st, ag, pull_gu ? SeqPull{h2_ptrs, B, Sl} : SeqPull{});
  g.scatter(hm, w_down, false, push_ptrs, static_cast<int>(S));
  sp.barrier();
  Tensor out = at::empty({Ml, H}, f32);
  ok(stb::launch_slot_sum_rmsnorm(recv.data_ptr<float>(), T, recv.stride(0),
                                  x_mid.data_ptr<float>(), out.data_ptr<float>(), nullptr, nullptr,
                                  nullptr, Ml, H, feps, st), "slot sum");
  return {inv1, qkv, attn, lse, x_mid, inv2, gu, out, hm};
}

// Backward of the layer above; uses 4 barrier epochs.  d_out / d_mid travel as bf16 through the
// peer-visible buffers dob_local / dmb_local; dX partial sums of the column-parallel GEMMs are
// scattered in fp32.
Tensor layer_backward_sp(
    const Tensor& d_out, const Tensor& x2, const Tensor& inv1, const Tensor& qkv,
    const Tensor& attn, const Tensor& lse, const Tensor& x_mid, const Tensor& inv2,
    const Tensor& gu, const Tensor& hm, const Tensor& w_qkv, const Tensor& w_o, const Tensor& w_gu,
    const Tensor& w_down, const Tensor& ln1, const Tensor& ln2, Tensor g_down, Tensor g_gate_up,
    Tensor g_ln2, Tensor g_o, Tensor g_bias, Tensor g_qkv, Tensor g_ln1, const Tensor& cos,
    const Tensor& sin, const c10::optional<Tensor>& positions, const c10::optional<Tensor>& mask,
    Tensor status, int64_t B, int64_t S, int64_t hq, int64_t hkv, Tensor dob_local,
    Tensor dmb_local, c10::ArrayRef<int64_t> h1_ptrs, c10::ArrayRef<int64_t> h2_ptrs,
    c10::ArrayRef<int64_t> dob_ptrs, c10::ArrayRef<int64_t> dmb_ptrs,
    c10::ArrayRef<int64_t> push_ptrs, Tensor recv, c10::ArrayRef<int64_t> flag_ptrs,
    int64_t tp_rank, int64_t epoch, int64_t flag_slot, int64_t wait_us, bool seq_pull) {
  const int64_t T = static_cast<int64_t>(h1_ptrs.size());
  const int64_t Sl = S / T, Ml = B * Sl, M = B * S, H = x2.size(1), D = 128;
  const int64_t W = (hq + 2 * hkv) * D, inter = w_down.size(1);
  auto bf = x2.options().dtype(at::kBFloat16);
  auto f32 = x2.options().dtype(at::kFloat);
  cudaStream_t st = at::cuda::getCurrentCUDAStream().stream();
  Gemm g{st, status.data_ptr<int>()};
  SpLink sp = make_link(st, g.status, flag_ptrs, tp_rank, epoch, flag_slot, wait_us);
  const int* pos = positions.has_value() ? positions->data_ptr<int>() : nullptr;
  const MaskView mv(mask);
  const uint8_t* km = mv.bytes;
  constexpr int kPartial = 592;

  ok(stb::launch_cast_f32_to_bf16(d_out.data_ptr<float>(), dob_local.data_ptr(), Ml * H, st), "cast");
  sp.barrier();
  Tensor d_full = at::empty({M, H}, bf), h_full = at::empty({M, H}, bf);
  Tensor d_hm = at::empty({M, inter}, bf);
  if (seq_pull) {
    // dX down gathers the peers' output-gradient slices while it runs; dW down reads them locally
    g.run(d_full, w_down, d_hm, false, true, nullptr, nullptr, SeqPull{dob_ptrs, B, Sl});
    g.run(d_full, hm, g_down, true, true, nullptr, nullptr);                // dW down
  } else {
    sp.gather(dob_ptrs, d_full, B, Sl);
    g.run(d_full, hm, g_down, true, true, nullptr, nullptr);                // dW down
    g.run(d_full, w_down, d_hm, false, true, nullptr, nullptr);             // dX down (local cols)
  }
  Tensor d_gu = at::empty({M, 2 * inter}, bf);
  ok(stb::launch_swiglu_bwd(d_hm.data_ptr(), gu.data_ptr(), d_gu.data_ptr(), M, inter, st), "swiglu_bwd");
  sp.gather(h2_ptrs, h_full, B, Sl);                                        // re-gather h2
  g.run(d_gu, h_full, g_gate_up, true, true, nullptr, nullptr);             // dW gate|up
  g.scatter(d_gu, w_gu, true, push_ptrs, static_cast<int>(S));              // dX gate|up partial
  sp.barrier();
  Tensor d_h2 = at::empty({Ml, H}, f32);
  ok(stb::launch_slot_sum_rmsnorm(recv.data_ptr<float>(), T, recv.stride(0), nullptr,
                                  d_h2.data_ptr<float>(), nullptr, nullptr, nullptr, Ml, H, 0.f, st),
     "slot sum");
  Tensor d_mid = at::empty({Ml, H}, f32), partial = at::empty({kPartial, H}, f32);
  ok(stb::launch_rmsnorm_bwd(d_h2.data_ptr<float>(), x_mid.data_ptr<float>(), ln2.data_ptr<float>(),
                             inv2.data_ptr<float>(), d_out.data_ptr<float>(), d_mid.data_ptr<float>(),
                             partial.data_ptr<float>(), kPartial, Ml, H, st), "rmsnorm_bwd");
  ok(stb::launch_colsum_f32(partial.data_ptr<float>(), g_ln2.data_ptr<float>(), kPartial, H, false, st), "colsum");

  ok(stb::launch_cast_f32_to_bf16(d_mid.data_ptr<float>(), dmb_local.data_ptr(), Ml * H, st), "cast");
  sp.barrier();
  Tensor d_attn = at::empty({M, hq * D}, bf);
  if (seq_pull) {
    g.run(d_full, w_o, d_attn, false, true, nullptr, nullptr, SeqPull{dmb_ptrs, B, Sl});  // dX o
    g.run(d_full, attn, g_o, true, true, nullptr, nullptr);                 // dW o
  } else {
    sp.gather(dmb_ptrs, d_full, B, Sl);
    g.run(d_full, attn, g_o, true, true, nullptr, nullptr);                 // dW o
    g.run(d_full, w_o, d_attn, false, true, nullptr, nullptr);              // dX o (local heads)
  }
  Tensor d_qkv = at::empty({M, W}, bf), delta = at::empty({B, hq, S}, f32);
  stb::AttnBwdCall bc{};
  bc.qkv = qkv.data_ptr();
  bc.out = attn.data_ptr();
  bc.dout = d_attn.data_ptr();
  bc.lse = lse.data_ptr<float>();
  bc.delta = delta.data_ptr<float>();
  bc.dqkv = d_qkv.data_ptr();
  const int parts = stb::attention_bwd_parts(static_cast<int>(B), static_cast<int>(S),
                                             static_cast<int>(hq), static_cast<int>(hkv));
  Tensor dkv_parts;
  if (parts > 1) dkv_parts = at::empty({parts, M, 2 * hkv * D}, f32);
  bc.dkv_accum = parts > 1 ? dkv_parts.data_ptr<float>() : nullptr;
  bc.dkv_accum_floats = parts > 1 ? dkv_parts.numel() : 0;
  bc.key_mask = km;
  bc.key_bits = mv.bits;
  bc.key_bits_pitch = mv.pitch;
  bc.batch = static_cast<int>(B);
  bc.seq = static_cast<int>(S);
  bc.hq = static_cast<int>(hq);
  bc.hkv = static_cast<int>(hkv);
  bc.scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(D)));
  ok(stb::launch_attention_bwd(bc, g.status, st), "attention_bwd");
  ok(stb::launch_rope(d_qkv.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), pos, M, S, hq,
                      hkv, D, true, st), "rope inverse");
  Tensor bias_partial = at::empty({64, W}, f32);
  ok(stb::launch_colsum_bf16(d_qkv.data_ptr(), W, g_bias.data_ptr<float>(), M, W, false,
                             bias_partial.data_ptr<float>(), 64, st), "bias colsum");
  sp.gather(h1_ptrs, h_full, B, Sl);                                        // re-gather h1
  g.run(d_qkv, h_full, g_qkv, true, true, nullptr, nullptr);                // dW q|k|v
  g.scatter(d_qkv, w_qkv, true, push_ptrs, static_cast<int>(S));            // dX q|k|v partial
  sp.barrier();
  Tensor d_h1 = at::empty({Ml, H}, f32);
  ok(stb::launch_slot_sum_rmsnorm(recv.data_ptr<float>(), T, recv.stride(0), nullptr,
                                  d_h1.data_ptr<float>(), nullptr, nullptr, nullptr, Ml, H, 0.f, st),
     "slot sum");
  Tensor dx = at::empty({Ml, H}, f32);
  ok(stb::launch_rmsnorm_bwd(d_h1.data_ptr<float>(), x2.data_ptr<float>(), ln1.data_ptr<float>(),
                             inv1.data_ptr<float>(), d_mid.data_ptr<float>(), dx.data_ptr<float>(),
                             partial.data_ptr<float>(), kPartial, Ml, H, st), "rmsnorm_bwd");
  ok(stb::launch_colsum_f32(partial.data_ptr<float>(), g_ln1.data_ptr<float>(), kPartial, H, false, st), "colsum");
  return dx;
}


// ---------------------------------------------------------------------------------------------
// Tensor parallel layer without sequence parallelism: activations are replicated over the TP
// group, column-parallel GEMMs need no communication, and the partial sums of the row-parallel
// GEMMs (forward o_proj / down_proj, backward dX of q|k|v and gate|up) are all-reduced: the GEMM
// epilogue pushes its fp32 rows into slot `tp_rank` of every member's receive set and the next
// kernel adds the T slots.  Two receive sets alternate, so one barrier per all-reduce is enough
// (a set is overwritten two all-reduces later, after a barrier that every reader has passed).
// push_a / push_b: per member, the address of this rank's slot in that member's set A / B.
// Uses 2 barrier epochs per call.
std::vector<Tensor> layer_forward_tp(
    const Tensor& x2, const Tensor& w_qkv, const Tensor& b_qkv, const Tensor& w_o,
    const Tensor& w_gu, const Tensor& w_down, const Tensor& ln1, const Tensor& ln2,
    const Tensor& cos, const Tensor& sin, const c10::optional<Tensor>& positions,
    const c10::optional<Tensor>& mask, Tensor status, int64_t B, int64_t S, int64_t hq,
    int64_t hkv, double eps, c10::ArrayRef<int64_t> push_a, c10::ArrayRef<int64_t> push_b,
    Tensor recv_a, Tensor recv_b, c10::ArrayRef<int64_t> flag_ptrs, int64_t tp_rank,
    int64_t epoch, int64_t flag_slot, int64_t wait_us, c10::ArrayRef<int64_t> ag_arenas,
    bool ag_wire_fp32, const c10::optional<Tensor>& ag_segs_qkv,
    const c10::optional<Tensor>& ag_segs_gu, const c10::optional<Tensor>& ag_full) {
  const AgPlan ag = make_ag_plan(ag_arenas, ag_wire_fp32, ag_segs_qkv, ag_segs_gu, ag_full);
  const int64_t T = static_cast<int64_t>(push_a.size());
  const int64_t M = B * S, H = x2.size(1), D = 128;
  const int64_t W = (hq + 2 * hkv) * D, inter = w_down.size(1);
  TORCH_CHECK(recv_a.dim() == 3 && recv_a.size(0) == T && recv_a.size(1) == M && recv_a.size(2) == H &&
                  recv_b.sizes() == recv_a.sizes(), "tensor-parallel layer: receive sets mismatch");
  auto bf = x2.options().dtype(at::kBFloat16);
  auto f32 = x2.options().dtype(at::kFloat);
  cudaStream_t st = at::cuda::getCurrentCUDAStream().stream();
  Gemm g{st, status.data_ptr<int>()};
  SpLink sp = make_link(st, g.status, flag_ptrs, tp_rank, epoch, flag_slot, wait_us);
  const int* pos = positions.has_value() ? positions->data_ptr<int>() : nullptr;
  const MaskView mv(mask);
  const uint8_t* km = mv.bytes;
  const float feps = static_cast<float>(eps);

  Tensor h1 = at::empty({M, H}, bf), inv1 = at::empty({M}, f32);
  ok(stb::launch_rmsnorm_fwd(x2.data_ptr<float>(), ln1.data_ptr<float>(), h1.data_ptr(),
                             inv1.data_ptr<float>(), M, H, feps, false, st), "rmsnorm");
  Tensor qkv = at::empty({M, W}, bf);
  g.qkv_proj(h1, w_qkv, qkv, b_qkv.data_ptr<float>(), ag);
  ok(stb::launch_rope(qkv.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), pos, M, S, hq,
                      hkv, D, false, st), "rope");
  Tensor attn = at::empty({M, hq * D}, bf), lse = at::empty({B, hq, S}, f32);
  stb::AttnCall ac{qkv.data_ptr(), attn.data_ptr(), lse.data_ptr<float>(), km, static_cast<int>(B),
                   static_cast<int>(S), static_cast<int>(hq), static_cast<int>(hkv),
                   static_cast<float>(1.0 / std::sqrt(static_cast<double>(D)))};
  ac.key_bits = mv.bits;
  ac.key_bits_pitch = mv.pitch;
  ok(stb::launch_attention_fwd(ac, g.status, st), "attention_fwd");
  g.broadcast(attn, w_o, false, push_a);
  sp.barrier();
  Tensor x_mid = at::empty({M, H}, f32), h2 = at::empty({M, H}, bf), inv2 = at::empty({M}, f32);
  ok(stb::launch_slot_sum_rmsnorm(recv_a.data_ptr<float>(), T, recv_a.stride(0),
                                  x2.data_ptr<float>(), x_mid.data_ptr<float>(),
                                  ln2.data_ptr<float>(), h2.data_ptr(), inv2.data_ptr<float>(), M, H,
                                  feps, st), "slot sum + rmsnorm");
  Tensor gu = at::empty({M, 2 * inter}, bf), hm = at::empty({M, inter}, bf);
  g.gate_up(h2, w_gu, gu, hm, st, ag);
  g.broadcast(hm, w_down, false, push_b);
  sp.barrier();
  Tensor out = at::empty({M, H}, f32);
  ok(stb::launch_slot_sum_rmsnorm(recv_b.data_ptr<float>(), T, recv_b.stride(0),
                                  x_mid.data_ptr<float>(), out.data_ptr<float>(), nullptr, nullptr,
                                  nullptr, M, H, feps, st), "slot sum");
  return {h1, inv1, qkv, attn, lse, x_mid, h2, inv2, gu, out, hm};
}


// Backward of the layer above (d_out is replicated over the TP group); 2 barrier epochs.
Tensor layer_backward_tp(
    const Tensor& d_out, const Tensor& x2, const Tensor& inv1, const Tensor& h1, const Tensor& qkv,
    const Tensor& attn, const Tensor& lse, const Tensor& x_mid, const Tensor& inv2, const Tensor& h2,
    const Tensor& gu, const Tensor& hm, const Tensor& w_qkv, const Tensor& w_o, const Tensor& w_gu,
    const Tensor& w_down, const Tensor& ln1, const Tensor& ln2, Tensor g_down, Tensor g_gate_up,
    Tensor g_ln2, Tensor g_o, Tensor g_bias, Tensor g_qkv, Tensor g_ln1, const Tensor& cos,
    const Tensor& sin, const c10::optional<Tensor>& positions, const c10::optional<Tensor>& mask,
    Tensor status, int64_t B, int64_t S, int64_t hq, int64_t hkv, c10::ArrayRef<int64_t> push_a,
    c10::ArrayRef<int64_t> push_b, Tensor recv_a, Tensor recv_b, c10::ArrayRef<int64_t> flag_ptrs,
    int64_t tp_rank, int64_t epoch, int64_t flag_slot, int64_t wait_us) {
  const int64_t T = static_cast<int64_t>(push_a.size());
  const int64_t M = B * S, H = x2.size(1), D = 128;
  const int64_t W = (hq + 2 * hkv) * D, inter = w_down.size(1);
  auto bf = x2.options().dtype(at::kBFloat16);
  auto f32 = x2.options().dtype(at::kFloat);
  cudaStream_t st = at::cuda::getCurrentCUDAStream().stream();
  Gemm g{st, status.data_ptr<int>()};
  SpLink sp = make_link(st, g.status, flag_ptrs, tp_rank, epoch, flag_slot, wait_us);
  const int* pos = positions.has_value() ? positions->data_ptr<int>() : nullptr;
  const MaskView mv(mask);
  const uint8_t* km = mv.bytes;
  constexpr int kPartial = 592;

  Tensor d_out_b = at::empty({M, H}, bf);
  ok(stb::launch_cast_f32_to_bf16(d_out.data_ptr<float>(), d_out_b.data_ptr(), M * H, st), "cast");
  g.run(d_out_b, hm, g_down, true, true, nullptr, nullptr);                 // dW down (local cols)
  Tensor d_hm = at::empty({M, inter}, bf);
  g.run(d_out_b, w_down, d_hm, false, true, nullptr, nullptr);              // dX down (local cols)
  Tensor d_gu = at::empty({M, 2 * inter}, bf);
  ok(stb::launch_swiglu_bwd(d_hm.data_ptr(), gu.data_ptr(), d_gu.data_ptr(), M, inter, st), "swiglu_bwd");
  g.run(d_gu, h2, g_gate_up, true, true, nullptr, nullptr);                 // dW gate|up
  g.broadcast(d_gu, w_gu, true, push_a);                                    // dX gate|up partial
  sp.barrier();
  Tensor d_h2 = at::empty({M, H}, f32);
  ok(stb::launch_slot_sum_rmsnorm(recv_a.data_ptr<float>(), T, recv_a.stride(0), nullptr,
                                  d_h2.data_ptr<float>(), nullptr, nullptr, nullptr, M, H, 0.f, st),
     "slot sum");
  Tensor d_mid = at::empty({M, H}, f32), partial = at::empty({kPartial, H}, f32);
  ok(stb::launch_rmsnorm_bwd(d_h2.data_ptr<float>(), x_mid.data_ptr<float>(), ln2.data_ptr<float>(),
                             inv2.data_ptr<float>(), d_out.data_ptr<float>(), d_mid.data_ptr<float>(),
                             partial.data_ptr<float>(), kPartial, M, H, st), "rmsnorm_bwd");
  ok(stb::launch_colsum_f32(partial.data_ptr<float>(), g_ln2.data_ptr<float>(), kPartial, H, false, st), "colsum");

  Tensor d_mid_b = at::empty({M, H}, bf);
  ok(stb::launch_cast_f32_to_bf16(d_mid.data_ptr<float>(), d_mid_b.data_ptr(), M * H, st), "cast");
  g.run(d_mid_b, attn, g_o, true, true, nullptr, nullptr);                  // dW o
  Tensor d_attn = at::empty({M, hq * D}, bf);
  g.run(d_mid_b, w_o, d_attn, false, true, nullptr, nullptr);               // dX o (local heads)
  Tensor d_qkv = at::empty({M, W}, bf), delta = at::empty({B, hq, S}, f32);
  stb::AttnBwdCall bc{};
  bc.qkv = qkv.data_ptr();
  bc.out = attn.data_ptr();
  bc.dout = d_attn.data_ptr();
  bc.lse = lse.data_ptr<float>();
  bc.delta = delta.data_ptr<float>();
  bc.dqkv = d_qkv.data_ptr();
  const int parts = stb::attention_bwd_parts(static_cast<int>(B), static_cast<int>(S),
                                             static_cast<int>(hq), static_cast<int>(hkv));
  Tensor dkv_parts;
  if (parts > 1) dkv_parts = at::empty({parts, M, 2 * hkv * D}, f32);
  bc.dkv_accum = parts > 1 ? dkv_parts.data_ptr<float>() : nullptr;
  bc.dkv_accum_floats = parts > 1 ? dkv_parts.numel() : 0;
  bc.key_mask = km;
  bc.key_bits = mv.bits;
  bc.key_bits_pitch = mv.pitch;
  bc.batch = static_cast<int>(B);
  bc.seq = static_cast<int>(S);
  bc.hq = static_cast<int>(hq);
  bc.hkv = static_cast<int>(hkv);
  bc.scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(D)));
  ok(stb::launch_attention_bwd(bc, g.status, st), "attention_bwd");
  ok(stb::launch_rope(d_qkv.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), pos, M, S, hq,
                      hkv, D, true, st), "rope inverse");
  Tensor bias_partial = at::empty({64, W}, f32);
  ok(stb::launch_colsum_bf16(d_qkv.data_ptr(), W, g_bias.data_ptr<float>(), M, W, false,
                             bias_partial.data_ptr<float>(), 64, st), "bias colsum");
  g.run(d_qkv, h1, g_qkv, true, true, nullptr, nullptr);                    // dW q|k|v
  g.broadcast(d_qkv, w_qkv, true, push_b);                                  // dX q|k|v partial
  sp.barrier();
  Tensor d_h1 = at::empty({M, H}, f32);
  ok(stb::launch_slot_sum_rmsnorm(recv_b.data_ptr<float>(), T, recv_b.stride(0), nullptr,
                                  d_h1.data_ptr<float>(), nullptr, nullptr, nullptr, M, H, 0.f, st),
     "slot sum");
  Tensor dx = at::empty({M, H}, f32);
  ok(stb::launch_rmsnorm_bwd(d_h1.data_ptr<float>(), x2.data_ptr<float>(), ln1.data_ptr<float>(),
                             inv1.data_ptr<float>(), d_mid.data_ptr<float>(), dx.data_ptr<float>(),
                             partial.data_ptr<float>(), kPartial, M, H, st), "rmsnorm_bwd");
  ok(stb::launch_colsum_f32(partial.data_ptr<float>(), g_ln1.data_ptr<float>(), kPartial, H, false, st), "colsum");
  return dx;
}

}  // namespace

// number of launch sequences currently held as graphs / drop all of them (and their buffers)
int64_t replay_graphs() { return static_cast<int64_t>(replay_cache().graphs()); }
void replay_clear() { replay_cache().clear(); }

TORCH_LIBRARY_FRAGMENT(stb, m) {
  m.def("layer_forward", &layer_forward);
  m.def("layer_backward", &layer_backward);
  m.def("layer_forward_sp", &layer_forward_sp);
  m.def("layer_backward_sp", &layer_backward_sp);
  m.def("layer_forward_tp", &layer_forward_tp);
  m.def("layer_backward_tp", &layer_backward_tp);
  m.def("replay_graphs", &replay_graphs);
  m.def("replay_clear", &replay_clear);
}
