// Allocation-free column sum (see noalloc.h for the contract and for who needs it).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "noalloc.h"

namespace {

constexpr int kPartialRows = 64;
constexpr int kMaxDevices = 64;

// The workspace lives in the library image: one copy per GPU that loads it.  In host code this
// name is only a handle for the runtime; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) float g_colsum_workspace[kPartialRows * STB_COLSUM_NOALLOC_MAX_COLS];

// partial[b, c] = sum of x[r, c] over the rows r = b, b + gridDim.y, ...   (two columns/thread)
__global__ void noalloc_partial_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                       float* __restrict__ partial, int rows, int cols) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= cols) return;
  float s0 = 0.f, s1 = 0.f;
  for (int r = blockIdx.y; r < rows; r += gridDim.y) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + r * ldx + c);
    const float2 f = __bfloat1622float2(v);
    s0 += f.x;
    s1 += f.y;
  }
  partial[static_cast<int64_t>(blockIdx.y) * cols + c] = s0;
  partial[static_cast<int64_t>(blockIdx.y) * cols + c + 1] = s1;
}

// out[c] (+)= sum_b partial[b, c], fixed order
__global__ void noalloc_final_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                     int cols, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int b = 0; b < kPartialRows; ++b) s += partial[static_cast<int64_t>(b) * cols + c];
  out[c] = accumulate ? out[c] + s : s;
}

float* g_workspace_address[kMaxDevices] = {};

}  // namespace

extern "C" int stb_colsum_bf16_noalloc(const void* x, int64_t ldx, float* out, int rows, int cols,
                                       int accumulate, void* stream) {
  if (x == nullptr || out == nullptr || rows <= 0 || cols <= 0 || (cols & 1) ||
      cols > STB_COLSUM_NOALLOC_MAX_COLS || ldx < cols || (ldx & 1))
    return -1;
  // the kernels read x two bf16 at a time (4-byte loads) and write fp32: a view that starts at an
  // odd element offset would be a misaligned device access, so it is refused here, unlaunched
  if ((reinterpret_cast<uintptr_t>(x) & 3) != 0 || (reinterpret_cast<uintptr_t>(out) & 3) != 0)
    return -1;
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (device < 0 || device >= kMaxDevices) return -1;
  if (g_workspace_address[device] == nullptr) {
    // once per device, with that device current: resolve the device address of the array
    float* address = nullptr;
    err = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_colsum_workspace);
    if (err != cudaSuccess) return static_cast<int>(err);
    g_workspace_address[device] = address;
  }
  float* workspace = g_workspace_address[device];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid((cols / 2 + 127) / 128, kPartialRows);
  noalloc_partial_kernel<<<grid, 128, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx, workspace,
                                              rows, cols);
  err = cudaGetLastError();
  if (err != cudaSuccess) return static_cast<int>(err);
  noalloc_final_kernel<<<(cols + 127) / 128, 128, 0, s>>>(workspace, out, cols, accumulate ? 1 : 0);
  err = cudaGetLastError();
  return err == cudaSuccess ? 0 : static_cast<int>(err);
}
