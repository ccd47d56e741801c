// Memory-bound kernels of the Qwen2 training step, written for HBM3e: one pass over the data,
// 16-byte accesses, fp32 math.  Each replaces an ATen chain of the reference
// (src/sharded_runtime/runtime/qwen2_operators.py:156-204, src/sharded_runtime/models/qwen2.py:123-159,
// 262-278, src/sharded_runtime/runtime/qwen2_adapter.py:248-273, src/sharded_runtime/training/qwen2_trainer.py:48).
#include <cuda_bf16.h>
#include <math.h>

#include "api.h"

namespace stb {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; every thread receives the result.  `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}

// ------------------------------------------------------------------ RMSNorm
// One CTA per row; x fp32 -> y = (x * rsqrt(mean(x^2)+eps)) * w, rounded once to the output type.
template <bool Y_FP32>
__global__ void rmsnorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                   void* __restrict__ y, float* __restrict__ inv_out, int cols,
                                   float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const float* xr = x + row * cols;
  float ss = 0.f;
  for (int c = threadIdx.x * 4; c < cols; c += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xr + c);
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / cols + eps);
  if (threadIdx.x == 0) inv_out[row] = inv;
  for (int c = threadIdx.x * 4; c < cols; c += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xr + c);
    const float4 g = *reinterpret_cast<const float4*>(w + c);
    const float a = v.x * inv * g.x, b = v.y * inv * g.y, cc = v.z * inv * g.z,
                d = v.w * inv * g.w;
    if (Y_FP32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + row * cols + c) =
          make_float4(a, b, cc, d);
    } else {
      uint2 pk;
      pk.x = pack2(a, b);
      pk.y = pack2(cc, d);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(y) + row * cols + c) = pk;
    }
  }
}

// Tail of a sequence reduce-scatter whose partial sums were pushed into `n_slots` receive slots
// (slot k at slots + k * slot_stride): sum_out = residual + sum_k slot_k, and, when a norm weight
// is given, y = bf16(rmsnorm(sum_out) * w) with the row's inverse RMS.  One CTA per row.
__global__ void slot_sum_rmsnorm_kernel(const float* __restrict__ slots, int n_slots,
                                        int64_t slot_stride, const float* __restrict__ residual,
                                        float* __restrict__ sum_out, const float* __restrict__ w,
                                        __nv_bfloat16* __restrict__ y, float* __restrict__ inv_out,
                                        int cols, float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int64_t off = row * cols;
  float ss = 0.f;
  for (int c = threadIdx.x * 4; c < cols; c += blockDim.x * 4) {
    float4 acc = residual ? *reinterpret_cast<const float4*>(residual + off + c)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < n_slots; ++k) {
      const float4 t = *reinterpret_cast<const float4*>(slots + k * slot_stride + off + c);
      acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
    }
    *reinterpret_cast<float4*>(sum_out + off + c) = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  if (w == nullptr) return;
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / cols + eps);
  if (threadIdx.x == 0) inv_out[row] = inv;
  for (int c = threadIdx.x * 4; c < cols; c += blockDim.x * 4) {
    // each thread re-reads exactly the elements it wrote above
    const float4 v = *reinterpret_cast<const float4*>(sum_out + off + c);
    const float4 g = *reinterpret_cast<const float4*>(w + c);
    uint2 pk;
    pk.x = pack2(v.x * inv * g.x, v.y * inv * g.y);
    pk.y = pack2(v.z * inv * g.z, v.w * inv * g.w);
    *reinterpret_cast<uint2*>(y + off + c) = pk;
  }
}

// dx = inv * (g*w - x * inv^2 * mean(g*w*x)) (+ incoming residual gradient);
// d(weight) partial per CTA = sum over its rows of g * (x*inv).  Rows are strided over CTAs.
__global__ void rmsnorm_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                   const float* __restrict__ w, const float* __restrict__ inv,
                                   const float* __restrict__ dres, float* __restrict__ dx,
                                   float* __restrict__ dw_partial, int rows, int cols) {
  extern __shared__ float sm[];  // cols floats of dw accumulation + 32 for reductions
  float* dw_acc = sm;
  float* red = sm + cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dw_acc[c] = 0.f;
  __syncthreads();
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * cols;
    const float* gr = dy + row * cols;
    const float iv = inv[row];
    float dot = 0.f;
    for (int c = threadIdx.x * 4; c < cols; c += blockDim.x * 4) {
      const float4 xv = *reinterpret_cast<const float4*>(xr + c);
      const float4 gv = *reinterpret_cast<const float4*>(gr + c);
      const float4 wv = *reinterpret_cast<const float4*>(w + c);
      dot += gv.x * wv.x * xv.x + gv.y * wv.y * xv.y + gv.z * wv.z * xv.z + gv.w * wv.w * xv.w;
    }
    dot = block_sum(dot, red);
    const float coef = iv * iv * dot / cols;
    for (int c = threadIdx.x * 4; c < cols; c += blockDim.x * 4) {
      const float4 xv = *reinterpret_cast<const float4*>(xr + c);
      const float4 gv = *reinterpret_cast<const float4*>(gr + c);
      const float4 wv = *reinterpret_cast<const float4*>(w + c);
      float4 o;
      o.x = iv * (gv.x * wv.x - xv.x * coef);
      o.y = iv * (gv.y * wv.y - xv.y * coef);
      o.z = iv * (gv.z * wv.z - xv.z * coef);
      o.w = iv * (gv.w * wv.w - xv.w * coef);
      if (dres != nullptr) {
        const float4 r = *reinterpret_cast<const float4*>(dres + row * cols + c);
        o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
      }
      *reinterpret_cast<float4*>(dx + row * cols + c) = o;
      // each thread owns fixed columns across rows, so no race on dw_acc
      dw_acc[c] += gv.x * xv.x * iv;
      dw_acc[c + 1] += gv.y * xv.y * iv;
      dw_acc[c + 2] += gv.z * xv.z * iv;
      dw_acc[c + 3] += gv.w * xv.w * iv;
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    dw_partial[static_cast<int64_t>(blockIdx.x) * cols + c] = dw_acc[c];
}

// out[c] (+)= sum_r partial[r, c]; deterministic order.
// out[c] = sum_r partial[r, c].  A CTA covers 32 columns with 8 row groups (blockDim 32 x 8): the
// groups stride over the rows, then combine through shared memory in a fixed order.
__global__ void colsum_f32_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                  int rows, int cols, int accumulate) {
  __shared__ float part[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < cols)
    for (int r = threadIdx.y; r < rows; r += 8) s += partial[static_cast<int64_t>(r) * cols + c];
  part[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) t += part[g][threadIdx.x];
    out[c] = accumulate ? out[c] + t : t;
  }
}

// scratch[b, c] = sum over the rows handled by CTA row-group b of x[r, c] (bf16 input).
__global__ void colsum_bf16_partial_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                           float* __restrict__ scratch, int rows, int cols) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= cols) return;
  float s0 = 0.f, s1 = 0.f;
  for (int r = blockIdx.y; r < rows; r += gridDim.y) {
    const float2 v = unpack2(*reinterpret_cast<const uint32_t*>(x + r * ldx + c));
    s0 += v.x;
    s1 += v.y;
  }
  scratch[static_cast<int64_t>(blockIdx.y) * cols + c] = s0;
  scratch[static_cast<int64_t>(blockIdx.y) * cols + c + 1] = s1;
}

// ------------------------------------------------------------------ RoPE
// rotate_half form: out[i] = x[i]*cos - x[i+d/2]*sin ; out[i+d/2] = x[i+d/2]*cos + x[i]*sin.
// Applied in place to the q and k heads of the packed qkv rows; `inverse` flips the sign of sin
// (the backward pass is the transposed rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ positions,
                            int rows, int seq, int hq, int hkv, int d, int inverse) {
  const int half = d / 2;
  const int heads = hq + hkv;
  const int pairs_per_row = heads * (half / 2);  // two (i, i+half) pairs per thread
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(rows) * pairs_per_row) return;
  const int row = static_cast<int>(idx / pairs_per_row);
  const int rem = static_cast<int>(idx % pairs_per_row);
  const int head = rem / (half / 2);
  const int i = (rem % (half / 2)) * 2;
  const int pos = positions ? positions[row] : (row % seq);
  const int64_t stride = static_cast<int64_t>(hq + 2 * hkv) * d;
  __nv_bfloat16* base = qkv + row * stride + static_cast<int64_t>(head) * d;
  const float2 lo = unpack2(*reinterpret_cast<uint32_t*>(base + i));
  const float2 hi = unpack2(*reinterpret_cast<uint32_t*>(base + i + half));
  const float c0 = cos_t[pos * half + i], c1 = cos_t[pos * half + i + 1];
  float s0 = sin_t[pos * half + i], s1 = sin_t[pos * half + i + 1];
  if (inverse) {
    s0 = -s0;
    s1 = -s1;
  }
  *reinterpret_cast<uint32_t*>(base + i) = pack2(lo.x * c0 - hi.x * s0, lo.y * c1 - hi.y * s1);
  *reinterpret_cast<uint32_t*>(base + i + half) =
      pack2(hi.x * c0 + lo.x * s0, hi.y * c1 + lo.y * s1);
}

// ------------------------------------------------------------------ SwiGLU
// gu = [gate | up] packed per row ([rows, 2*inter]); h = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ h, int rows, int inter) {
  const int64_t n8 = static_cast<int64_t>(rows) * (inter / 8);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / (inter / 8);
    const int c = static_cast<int>(i % (inter / 8)) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + row * 2 * inter + c);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + row * 2 * inter + inter + c);
    const uint32_t* gp = reinterpret_cast<const uint32_t*>(&g);
    const uint32_t* up = reinterpret_cast<const uint32_t*>(&u);
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 gv = unpack2(gp[j]);
      const float2 uv = unpack2(up[j]);
      // match the reference rounding: silu(gate) is rounded to bf16 before the product
      const float sa = __bfloat162float(__float2bfloat16(gv.x / (1.f + __expf(-gv.x))));
      const float sb = __bfloat162float(__float2bfloat16(gv.y / (1.f + __expf(-gv.y))));
      op[j] = pack2(sa * uv.x, sb * uv.y);
    }
    *reinterpret_cast<uint4*>(h + row * inter + c) = o;
  }
}

// d(gate) = dh * up * (sig + gate*sig*(1-sig)), d(up) = dh * silu(gate).
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dh,
                                  const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, int rows, int inter) {
  const int64_t n8 = static_cast<int64_t>(rows) * (inter / 8);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / (inter / 8);
    const int c = static_cast<int>(i % (inter / 8)) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + row * 2 * inter + c);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + row * 2 * inter + inter + c);
    const uint4 d = *reinterpret_cast<const uint4*>(dh + row * inter + c);
    const uint32_t* gp = reinterpret_cast<const uint32_t*>(&g);
    const uint32_t* up = reinterpret_cast<const uint32_t*>(&u);
    const uint32_t* dp = reinterpret_cast<const uint32_t*>(&d);
    uint4 og, ou;
    uint32_t* ogp = reinterpret_cast<uint32_t*>(&og);
    uint32_t* oup = reinterpret_cast<uint32_t*>(&ou);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 gv = unpack2(gp[j]);
      const float2 uv = unpack2(up[j]);
      const float2 dv = unpack2(dp[j]);
      const float s0 = 1.f / (1.f + __expf(-gv.x)), s1 = 1.f / (1.f + __expf(-gv.y));
      ogp[j] = pack2(dv.x * uv.x * (s0 + gv.x * s0 * (1.f - s0)),
                     dv.y * uv.y * (s1 + gv.y * s1 * (1.f - s1)));
      oup[j] = pack2(dv.x * gv.x * s0, dv.y * gv.y * s1);
    }
    *reinterpret_cast<uint4*>(dgu + row * 2 * inter + c) = og;
    *reinterpret_cast<uint4*>(dgu + row * 2 * inter + inter + c) = ou;
  }
}

// ------------------------------------------------------------------ vocabulary cross-entropy
// One CTA per row over bf16 logits: online log-sum-exp in fp32, loss_row = lse - logit[label]
// (0 when label == -100).
__global__ void ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, int64_t ld,
                              const int64_t* __restrict__ labels, float* __restrict__ lse_out,
                              float* __restrict__ loss_rows, int vocab) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x * 8; c < vocab; c += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(lr + c);
    const uint32_t* vp = reinterpret_cast<const uint32_t*>(&v);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = unpack2(vp[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  const float gmax = block_max(m, red);
  const float part = (m == -INFINITY) ? 0.f : s * __expf(m - gmax);
  const float tot = block_sum(part, red);
  if (threadIdx.x == 0) {
    const float lse = gmax + logf(tot);
    lse_out[row] = lse;
    const int64_t lab = labels[row];
    loss_rows[row] = (lab < 0) ? 0.f : lse - __bfloat162float(lr[lab]);
  }
}

// logits <- scale * (softmax(logits) - onehot(label)) in place (zero for ignored rows).
__global__ void ce_bwd_kernel(__nv_bfloat16* __restrict__ logits, int64_t ld,
                              const int64_t* __restrict__ labels, const float* __restrict__ lse,
                              const float* __restrict__ scale, int vocab) {
  const int64_t row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const int64_t lab = labels[row];
  const float sc = (lab < 0) ? 0.f : *scale;
  const float l = lse[row];
  for (int c = threadIdx.x * 8; c < vocab; c += blockDim.x * 8) {
    uint4 v = *reinterpret_cast<const uint4*>(lr + c);
    uint32_t* vp = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = unpack2(vp[j]);
      float a = __expf(t.x - l), b = __expf(t.y - l);
      if (c + 2 * j == lab) a -= 1.f;
      if (c + 2 * j + 1 == lab) b -= 1.f;
      vp[j] = pack2(a * sc, b * sc);
    }
    *reinterpret_cast<uint4*>(lr + c) = v;
  }
}

// Single-CTA deterministic sum (used for the per-row losses).
__global__ void sum_f32_kernel(const float* __restrict__ x, float* __restrict__ out, int n,
                               int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) *out = accumulate ? *out + s : s;
}

// ------------------------------------------------------------------ embedding backward
__global__ void embedding_scatter_add_kernel(const float* __restrict__ dx,
                                             const int64_t* __restrict__ ids,
                                             float* __restrict__ dw, int rows, int cols,
                                             int64_t vocab, int64_t pad_id) {
  const int64_t row = blockIdx.x;
  const int64_t id = ids[row];
  if (id < 0 || id >= vocab || id == pad_id) return;
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    atomicAdd(dw + id * cols + c, dx[row * cols + c]);
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                     int64_t n) {
  const int64_t n4 = n / 4;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float4 v = *reinterpret_cast<const float4*>(x + i * 4);
    uint2 pk;
    pk.x = pack2(v.x, v.y);
    pk.y = pack2(v.z, v.w);
    *reinterpret_cast<uint2*>(y + i * 4) = pk;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const int64_t i = n4 * 4 + threadIdx.x;
    y[i] = __float2bfloat16(x[i]);
  }
}

__global__ void add_f32_kernel(const float* __restrict__ a, const float* __restrict__ b,
                               float* __restrict__ o, int64_t n) {
  for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x * 4) {
    if (i + 3 < n) {
      const float4 x = *reinterpret_cast<const float4*>(a + i);
      const float4 y = *reinterpret_cast<const float4*>(b + i);
      *reinterpret_cast<float4*>(o + i) = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    } else {
      for (int64_t j = i; j < n; ++j) o[j] = a[j] + b[j];
    }
  }
}

// ------------------------------------------------------------------ optimisers
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v, int64_t n,
                             AdamWArgs a) {
  const float step_size = a.lr / a.bias_correction1;
  const float inv_bc2_sqrt = rsqrtf(a.bias_correction2);
  for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x * 4) {
    if (i + 3 < n) {
      float4 pv = *reinterpret_cast<float4*>(p + i);
      float4 gv = *reinterpret_cast<const float4*>(g + i);
      float4 mv = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      float* pp = &pv.x;
      float* gp = &gv.x;
      float* mp = &mv.x;
      float* vp = &vv.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gr = gp[j] * a.grad_scale;
        pp[j] *= 1.f - a.lr * a.weight_decay;
        mp[j] = a.beta1 * mp[j] + (1.f - a.beta1) * gr;
        vp[j] = a.beta2 * vp[j] + (1.f - a.beta2) * gr * gr;
        const float denom = sqrtf(vp[j]) * inv_bc2_sqrt + a.eps;
        pp[j] -= step_size * mp[j] / denom;
      }
      *reinterpret_cast<float4*>(p + i) = pv;
      *reinterpret_cast<float4*>(m + i) = mv;
      *reinterpret_cast<float4*>(v + i) = vv;
    } else {
      for (int64_t j = i; j < n; ++j) {
        const float gr = g[j] * a.grad_scale;
        float pj = p[j] * (1.f - a.lr * a.weight_decay);
        const float mj = a.beta1 * m[j] + (1.f - a.beta1) * gr;
        const float vj = a.beta2 * v[j] + (1.f - a.beta2) * gr * gr;
        pj -= step_size * mj / (sqrtf(vj) * inv_bc2_sqrt + a.eps);
        p[j] = pj;
        m[j] = mj;
        v[j] = vj;
      }
    }
  }
}

__global__ void sgd_kernel(float* __restrict__ p, const float* __restrict__ g, int64_t n,
                           float lr) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    p[i] -= lr * g[i];
}

// flags[0]: non-finite gradient seen; flags[1]: non-zero value inside a padding range.
__global__ void grad_check_kernel(const float* __restrict__ g, int64_t n,
                                  const int64_t* __restrict__ pad_ranges, int n_ranges,
                                  int* __restrict__ flags) {
  int bad = 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    bad |= !isfinite(g[i]);
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(&flags[0], 1);
  int padbad = 0;
  for (int r = blockIdx.x; r < n_ranges; r += gridDim.x) {
    const int64_t b = pad_ranges[2 * r], e = pad_ranges[2 * r + 1];
    for (int64_t i = b + threadIdx.x; i < e; i += blockDim.x) padbad |= (g[i] != 0.f);
  }
  if (__syncthreads_or(padbad) && threadIdx.x == 0) atomicOr(&flags[1], 1);
}

// cap = 0: eight CTAs per SM of the current device
inline int grid_for(int64_t work, int threads, int cap = 0) {
  if (cap <= 0) cap = sm_count() * 8;
  int64_t g = (work + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return static_cast<int>(g);
}

}  // namespace

// ----------------------------------------------------------------------------- NCCL-path packing
// The library all-gather / reduce-scatter of the portable path work on one packed buffer per
// unit: `degree` rank slots of `slot` elements, parameter p's shard at [start_p, start_p + q_p)
// of every slot.  One launch per unit moves all its parameters (table rows: start, q, numel,
// offset in the flat output).
__global__ void unpack_gathered_kernel(const float* __restrict__ packed, int64_t slot,
                                       const int64_t* __restrict__ table, float* __restrict__ out) {
  const int64_t* row = table + 4 * blockIdx.y;
  const int64_t start = row[0], q = row[1], numel = row[2], off = row[3];
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < numel; i += stride) {
    const int64_t r = i / q;
    out[off + i] = packed[r * slot + start + (i - r * q)];
  }
}

// Full gradients (one pointer per parameter) -> destination-major reduce-scatter input with zero
// padding.  blockIdx.y == n_params clears the unused tail [used, slot) of every rank slot.
__global__ void pack_gradients_kernel(const int64_t* __restrict__ grads,
                                      const int64_t* __restrict__ table, int n_params, int degree,
                                      int64_t slot, int64_t used, float* __restrict__ packed) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (static_cast<int>(blockIdx.y) == n_params) {
    const int64_t pad = slot - used;
    for (int64_t i = first; i < pad * degree; i += stride) {
      const int64_t r = i / pad;
      packed[r * slot + used + (i - r * pad)] = 0.f;
    }
    return;
  }
  const int64_t* row = table + 4 * blockIdx.y;
  const int64_t start = row[0], q = row[1], numel = row[2];
  const float* g = reinterpret_cast<const float*>(grads[blockIdx.y]);
  for (int64_t i = first; i < q * degree; i += stride) {
    const int64_t r = i / q;
    packed[r * slot + start + (i - r * q)] = i < numel ? g[i] : 0.f;
  }
}

cudaError_t launch_rmsnorm_fwd(const float* x, const float* w, void* y, float* inv, int rows,
                               int cols, float eps, bool y_fp32, cudaStream_t s) {
  if (cols % 4) return cudaErrorInvalidValue;
  const int threads = cols >= 1024 ? 256 : 128;
  if (y_fp32) {
    rmsnorm_fwd_kernel<true><<<rows, threads, 0, s>>>(x, w, y, inv, cols, eps);
    count_launch();
  } else {
    rmsnorm_fwd_kernel<false><<<rows, threads, 0, s>>>(x, w, y, inv, cols, eps);
    count_launch();
  }
  return cudaGetLastError();
}

cudaError_t launch_slot_sum_rmsnorm(const float* slots, int n_slots, int64_t slot_stride,
                                    const float* residual, float* sum_out, const float* w, void* y,
                                    float* inv, int rows, int cols, float eps, cudaStream_t s) {
  if (cols % 4 || n_slots < 1 || slot_stride % 4 || (w != nullptr && (y == nullptr || inv == nullptr)))
    return cudaErrorInvalidValue;
  const int threads = cols >= 1024 ? 256 : 128;
  slot_sum_rmsnorm_kernel<<<rows, threads, 0, s>>>(slots, n_slots, slot_stride, residual, sum_out, w,
                                                   reinterpret_cast<__nv_bfloat16*>(y), inv, cols,
                                                   eps);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_rmsnorm_bwd(const float* dy, const float* x, const float* w, const float* inv,
                               const float* dres_in, float* dx_out, float* dw_partial,
                               int partial_rows, int rows, int cols, cudaStream_t s) {
  if (cols % 4 || partial_rows < 1) return cudaErrorInvalidValue;
  const int threads = 256;
  const size_t smem = (cols + 32) * sizeof(float);
  rmsnorm_bwd_kernel<<<partial_rows, threads, smem, s>>>(dy, x, w, inv, dres_in, dx_out,
                                                         dw_partial, rows, cols);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_colsum_f32(const float* partial, float* out, int rows, int cols,
                              bool accumulate, cudaStream_t s) {
  colsum_f32_kernel<<<(cols + 31) / 32, dim3(32, 8), 0, s>>>(partial, out, rows, cols, accumulate);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_colsum_bf16(const void* x, int64_t ldx, float* out, int rows, int cols,
                               bool accumulate, float* scratch, int scratch_rows, cudaStream_t s) {
  if (cols % 2 || scratch_rows < 1) return cudaErrorInvalidValue;
  dim3 grid((cols / 2 + 127) / 128, scratch_rows);
  colsum_bf16_partial_kernel<<<grid, 128, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx,
                                                  scratch, rows, cols);
  count_launch();
  colsum_f32_kernel<<<(cols + 31) / 32, dim3(32, 8), 0, s>>>(scratch, out, scratch_rows, cols,
                                                             accumulate);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_rope(void* qkv, const float* cos, const float* sin, const int* positions,
                        int rows, int seq, int hq, int hkv, int d, bool inverse, cudaStream_t s) {
  if (d % 4) return cudaErrorInvalidValue;
  const int64_t work = static_cast<int64_t>(rows) * (hq + hkv) * (d / 4);
  rope_kernel<<<static_cast<int>((work + 255) / 256), 256, 0, s>>>(
      reinterpret_cast<__nv_bfloat16*>(qkv), cos, sin, positions, rows, seq, hq, hkv, d, inverse);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_swiglu_fwd(const void* gu, void* h, int rows, int inter, cudaStream_t s) {
  if (inter % 8) return cudaErrorInvalidValue;
  const int64_t work = static_cast<int64_t>(rows) * (inter / 8);
  swiglu_fwd_kernel<<<grid_for(work, 256, sm_count() * 16), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(gu), reinterpret_cast<__nv_bfloat16*>(h), rows, inter);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_swiglu_bwd(const void* dh, const void* gu, void* dgu, int rows, int inter,
                              cudaStream_t s) {
  if (inter % 8) return cudaErrorInvalidValue;
  const int64_t work = static_cast<int64_t>(rows) * (inter / 8);
  swiglu_bwd_kernel<<<grid_for(work, 256, sm_count() * 16), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(dh), reinterpret_cast<const __nv_bfloat16*>(gu),
      reinterpret_cast<__nv_bfloat16*>(dgu), rows, inter);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_ce_fwd(const void* logits, int64_t ld, const int64_t* labels, float* lse,
                          float* loss_rows, int rows, int vocab, cudaStream_t s) {
  if (vocab % 8 || ld % 8) return cudaErrorInvalidValue;
  ce_fwd_kernel<<<rows, 512, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, labels,
                                     lse, loss_rows, vocab);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_ce_bwd(void* logits, int64_t ld, const int64_t* labels, const float* lse,
                          const float* scale, int rows, int vocab, cudaStream_t s) {
  if (vocab % 8 || ld % 8) return cudaErrorInvalidValue;
  ce_bwd_kernel<<<rows, 512, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(logits), ld, labels, lse,
                                     scale, vocab);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_sum_f32(const float* x, float* out, int n, bool accumulate, cudaStream_t s) {
  sum_f32_kernel<<<1, 1024, 0, s>>>(x, out, n, accumulate);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_embedding_scatter_add(const float* dx, const int64_t* ids, float* dw, int rows,
                                         int cols, int64_t vocab, int64_t pad_id, cudaStream_t s) {
  embedding_scatter_add_kernel<<<rows, 256, 0, s>>>(dx, ids, dw, rows, cols, vocab, pad_id);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_cast_f32_to_bf16(const float* x, void* y, int64_t n, cudaStream_t s) {
  cast_f32_bf16_kernel<<<grid_for(n / 4 + 1, 256, sm_count() * 16), 256, 0, s>>>(
      x, reinterpret_cast<__nv_bfloat16*>(y), n);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_add_f32(const float* a, const float* b, float* out, int64_t n, cudaStream_t s) {
  add_f32_kernel<<<grid_for(n / 4 + 1, 256, sm_count() * 16), 256, 0, s>>>(a, b, out, n);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_adamw(float* p, const float* g, float* m, float* v, int64_t n, AdamWArgs a,
                         cudaStream_t s) {
  adamw_kernel<<<grid_for(n / 4 + 1, 256, sm_count() * 16), 256, 0, s>>>(p, g, m, v, n, a);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_sgd(float* p, const float* g, int64_t n, float lr, cudaStream_t s) {
  sgd_kernel<<<grid_for(n, 256, sm_count() * 16), 256, 0, s>>>(p, g, n, lr);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_grad_check(const float* g, int64_t n, const int64_t* pad_ranges, int n_ranges,
                              int* flags, cudaStream_t s) {
  grad_check_kernel<<<grid_for(n, 256, sm_count() * 8), 256, 0, s>>>(g, n, pad_ranges, n_ranges, flags);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_unpack_gathered(const float* packed, int64_t slot, const int64_t* table,
                                   int n_params, int64_t largest, float* out, cudaStream_t s) {
  if (n_params < 1 || slot < 1) return cudaErrorInvalidValue;
  dim3 grid(grid_for(largest, 256, sm_count() * 4), n_params);
  unpack_gathered_kernel<<<grid, 256, 0, s>>>(packed, slot, table, out);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_pack_gradients(const int64_t* grads, const int64_t* table, int n_params, int degree,
                                  int64_t slot, int64_t used, int64_t largest, float* packed,
                                  cudaStream_t s) {
  if (n_params < 1 || degree < 1 || slot < used) return cudaErrorInvalidValue;
  dim3 grid(grid_for(largest * degree, 256, sm_count() * 4), n_params + 1);
  pack_gradients_kernel<<<grid, 256, 0, s>>>(grads, table, n_params, degree, slot, used, packed);
  count_launch();
  return cudaGetLastError();
}

}  // namespace stb
