// Column sums of a bf16 matrix for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project.  It exists for hosts that embed
// this library where cudaMalloc / cudaFree (and therefore torch's allocator) are off limits while
// they run: code executing inside a region that forbids allocation (for instance between the
// begin and end of a stream capture owned by someone else), real-time loops with a fixed memory
// budget, or plugins loaded by a process that pre-partitioned the whole device.  The regular op
// (`torch.ops.stb.colsum_bf16`) takes its partial-sum workspace from the caller; this variant
// keeps that workspace in a fixed array inside the library instead.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest matrix width the built-in workspace covers (64 partial rows x 8192 columns of fp32 =
// 2 MiB of device memory, held by every GPU that loads the library until the process exits).
#define STB_COLSUM_NOALLOC_MAX_COLS 8192

// out[c] (+)= sum over rows r of x[r, c], x row-major bf16 with leading dimension ldx (elements),
// out fp32 [cols].  `stream` is a cudaStream_t (0 = default stream).  Enqueues two kernels and
// returns without synchronising.
//
// Alignment: x must be 4-byte aligned (the kernel loads two bf16 per access), so cols and ldx
// must be even and a view may not start at an odd element offset of its storage; out must be
// 4-byte aligned.
//
// Returns 0 on success; -1 for cols > STB_COLSUM_NOALLOC_MAX_COLS, odd cols, odd ldx, ldx < cols,
// non-positive sizes, null pointers, or a misaligned x / out (nothing is launched in any of these
// cases); otherwise the positive cudaError_t value of the failing runtime call.
//
// * Allocation: none -- no cudaMalloc, cudaFree, or allocating library routine is called.
// * First call on a device: looks up the device address of the workspace once (a host-side
//   runtime query, no launch) and caches it for that device.  Make that first call outside any
//   stream capture.
// * The workspace is shared by every call on the device and keeps the previous call's partial
//   sums.  Nothing has to start from zero: each call overwrites every cell it later reads.
//   Two calls that overlap on the GPU (different streams, no ordering between them) race on it;
//   order them with events or use one stream.
int stb_colsum_bf16_noalloc(const void* x, int64_t ldx, float* out, int rows, int cols,
                            int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
