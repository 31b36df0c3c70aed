// Arguments of the absorbed-MLA paged attention entry points (mla.cu: mma.sync kernel for any row
// count; mla_tc.cu: tcgen05 / TMEM kernel for decode rows). Shared so that both launchers and the
// Python binding agree on one layout.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

struct MbMlaArgs {
  const void* q;
  const void* cache;
  const int* block_table;
  int max_blocks;
  const int* q_start;
  const int* q_len;
  const int* ctx_len;
  const int* row_seq;        // [total_rows] sequence index of every query row (merge kernel)
  int num_seqs, max_q_len, max_ctx, total_rows;
  int H, block_size;
  long long num_blocks;
  float scale;
  float* out;
  void* ws;
  size_t ws_bytes;
  int part_tokens;           // 0 = default 1024
  uint32_t* status;
  int impl;                  // 0 = choose, 1 = mma.sync kernel, 2 = tcgen05 kernel (decode rows, H <= 128)
};

extern "C" int mb_mla_decode_tc(const MbMlaArgs* a, cudaStream_t stream);
