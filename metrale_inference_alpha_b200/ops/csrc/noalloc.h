// Allocation-free GEMM entry point. This has no counterpart in the reference engine: it
// exists for callers of this library that are not allowed to allocate device memory
// (code inside a stream capture, plugins embedded in another framework's memory plan,
// allocator-free real-time loops).
//
//   int mb_gemm_noalloc(const MbGemmArgs* args, cudaStream_t stream);
//
// Same arguments and result as mb_gemm (see gemm_tcgen05.cu), except that `ws`, `ws_bytes`
// and the tensor-parallel fields are ignored: the split-K workspace is a static device array
// of MB_NOALLOC_SCRATCH_BYTES inside the library (resident on every GPU that loads the
// library, until the process exits). Returns MB_ERR_TOO_LARGE (-3) when
// counters + tiles * splits * token_tile * 128 * 4 bytes exceeds that size.
// The first call on a device resolves the array's device address, zeroes the counters and
// waits for that (a stream synchronisation, once per device, serialised between threads by a
// lock); make it before starting a stream capture. Calls that overlap on the GPU race on the
// array. The argument block is defined in gemm_args.h.
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include "gemm_args.h"

#ifndef MB_NOALLOC_SCRATCH_BYTES
#define MB_NOALLOC_SCRATCH_BYTES (16u * 1024u * 1024u)
#endif

extern "C" int mb_gemm_noalloc(const MbGemmArgs* args, cudaStream_t stream);
