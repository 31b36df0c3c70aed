// Argument block of the tcgen05 GEMM launchers (mb_gemm, mb_gemm_noalloc): one definition
// shared by the kernel file, by C / C++ callers and mirrored field for field by the ctypes
// binding (ops/_native.py::GemmArgs).
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

// kernel selection (MbGemmArgs::flags)
#define MB_GEMM_ONE_TILE_PER_CTA 16     // never use the persistent kernel
#define MB_GEMM_DECODE_TILE_ORDER 64    // prefill-sized GEMMs keep the decode launch order (weight tiles in x)
#define MB_GEMM_PERSISTENT_PREFILL 128  // several 128-token tiles may run on the persistent kernel
#define MB_GEMM_GROUPED_ONE_CTA 512     // grouped GEMMs of small token tiles keep one CTA per SM (default: two)
#define MB_GEMM_DSMEM_SPLITK 256        // cluster split-K exchanges partial tiles over distributed shared memory
                                        // (default: through the L2-resident workspace)

struct MbGemmArgs {
  int kind, M, N, K, ldo, a_ld;
  const void* W;
  const void* X;
  void* out;
  const void* residual;
  const float* w_scale;
  const float* a_scale;
  float alpha;
  const void* sfa;
  const void* sfb;
  int sf_k64;
  int epilogue, out_f32;
  void* ws;
  size_t ws_bytes;
  uint32_t* status;
  int force_tn, force_splits, sm_count;
  int flags;                // MB_GEMM_* kernel-selection bits (0 = the defaults)
  long long* timing_trace;  // only read by builds with MB_GEMM_TIMING_EXPERIMENTS; leave null
  int no_cluster;           // keep split-K on the workspace path
  // quantised SwiGLU output (served by the persistent kernel only; MB_ERR_UNSUPPORTED otherwise)
  void* outq;
  int ldq;
  void* outq_sf;
  int outq_sf_k64;
  float outq_gs;
  const int* tile_expert;   // grouped mode (all four set together)
  const int* tile_row0;
  const int* tile_nrows;
  int n_per_expert, max_tiles;
};

extern "C" int mb_gemm(const MbGemmArgs* args, cudaStream_t stream);
