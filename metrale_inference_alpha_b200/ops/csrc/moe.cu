// Mixture-of-experts support kernels (the expert FFN itself is the grouped mode of the
// tcgen05 GEMM in gemm_tcgen05.cu).
//
//   mb_moe_route    one warp per token over <= 512 expert logits: softmax top-k, or sigmoid
//                   scores + selection bias with group-limited selection (keep the
//                   `topk_group` groups with the largest sum of their two best biased scores,
//                   then top-k inside them). Ties resolve to the lower expert id. Weights are
//                   the un-biased scores, optionally sum-normalised and scaled.
//   mb_moe_sort     counting sort of the (token, slot) pairs by *local* expert: per-expert row
//                   ranges, the pair -> row map, and a tile work-list of (expert, first row,
//                   rows) entries for the grouped GEMM. Pairs routed to experts outside
//                   [expert_lo, expert_lo + num_local) are dropped (expert parallelism).
//   mb_moe_gather   expert-sorted copy of activation rows (+ per-row / per-group scales).
//   mb_moe_combine  out[t] = sum_j w[t, j] * y[row(t, j)] (+ optional addend), fp32 math.
//
// Reference behaviour covered: kernels/gb10/common/moe_topk.cu, moe_topk_sigmoid.cu (no
// group limit there), moe_permute.cu (sort_by_expert, build_tile_worklist, permute_tokens,
// unpermute_reduce), moe_unpermute_blend.cu.
#include "common.cuh"

namespace {

constexpr int kMaxPerLane = 16;  // 512 experts / 32 lanes

__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ logits, long long ld, int T, int E, int K, int mode,
             const float* __restrict__ bias, int n_group, int topk_group, int renorm, float scaling,
             float* __restrict__ out_w, int* __restrict__ out_id, int out_ld, int shared_id, int gate_col) {
  const int tok = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (tok >= T) return;
  const float* x = logits + (size_t)tok * ld;
  float score[kMaxPerLane], sel[kMaxPerLane];
  const int per = (E + 31) / 32;
  // expert e = j * 32 + lane (interleaved so warp reductions see a whole 32-expert stripe)
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int e = j * 32 + lane;
    score[j] = (j < per && e < E) ? x[e] : -INFINITY;
    mx = fmaxf(mx, score[j]);
  }
  if (mode == 0) {  // softmax
    mx = mb::warp_max(mx);
    float se = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      score[j] = score[j] == -INFINITY ? 0.f : __expf(score[j] - mx);
      se += score[j];
    }
    se = mb::warp_sum(se);
    const float inv = 1.f / se;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = j * 32 + lane;
      score[j] *= inv;
      sel[j] = (j < per && e < E) ? score[j] : -INFINITY;
    }
  } else {          // sigmoid + selection bias
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = j * 32 + lane;
      const bool ok = j < per && e < E;
      score[j] = ok ? 1.f / (1.f + __expf(-score[j])) : 0.f;
      sel[j] = ok ? score[j] + (bias ? bias[e] : 0.f) : -INFINITY;
    }
    if (n_group > 1) {
      // group g owns experts [g * gs, (g + 1) * gs); score = sum of its two best sel values
      const int gs = E / n_group;
      float gscore_mine = -INFINITY;  // lane g (< n_group) keeps group g's score
      for (int g = 0; g < n_group; ++g) {
        float b1 = -INFINITY, b2 = -INFINITY;
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
          const int e = j * 32 + lane;
          if (j < per && e >= g * gs && e < (g + 1) * gs) {
            const float v = sel[j];
            if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
          }
        }
        // merge (b1, b2) pairs across lanes
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float o1 = __shfl_xor_sync(0xffffffffu, b1, o), o2 = __shfl_xor_sync(0xffffffffu, b2, o);
          const float n1 = fmaxf(b1, o1);
          const float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
          b1 = n1; b2 = n2;
        }
        if (lane == g) gscore_mine = b1 + b2;
      }
      // pick topk_group groups (ties -> lower group id); keep-mask as a bit set
      uint32_t keep = 0;
      for (int r = 0; r < topk_group; ++r) {
        float v = (lane < n_group && !((keep >> lane) & 1)) ? gscore_mine : -INFINITY;
        int idx = lane;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, v, o);
          const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
          if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        keep |= 1u << idx;
      }
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j) {
        const int e = j * 32 + lane;
        if (j < per && e < E && !((keep >> (e / gs)) & 1)) sel[j] = -INFINITY;
      }
    }
  }
  // iterative top-k over sel; weights come from score
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int r = 0; r < K; ++r) {
    float v = -INFINITY;
    int idx = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = j * 32 + lane;
      if (j < per && e < E && (sel[j] > v || (sel[j] == v && e < idx))) { v = sel[j]; idx = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    // owner lane reports the weight and retires the expert
    float w = 0.f;
    if ((idx & 31) == lane) {
      const int j = idx >> 5;
#pragma unroll
      for (int jj = 0; jj < kMaxPerLane; ++jj)
        if (jj == j) { w = score[jj]; sel[jj] = -INFINITY; }
    }
    w = __shfl_sync(0xffffffffu, w, idx & 31);
    wsum += w;
    if (lane == r) { my_w = w; my_id = idx; }
  }
  if (lane < K) {
    float w = my_w;
    if (renorm) w = w / (wsum + (mode == 0 ? 0.f : 1e-20f));
    out_w[(size_t)tok * out_ld + lane] = w * scaling;
    out_id[(size_t)tok * out_ld + lane] = my_id;
  }
  // an always-selected shared expert rides along as slot K: its weight is 1 or the sigmoid of an
  // extra logit column (the shared-expert gate row appended to the router weight)
  if (shared_id >= 0 && lane == K) {
    out_w[(size_t)tok * out_ld + K] = gate_col >= 0 ? 1.f / (1.f + __expf(-x[gate_col])) : 1.f;
    out_id[(size_t)tok * out_ld + K] = shared_id;
  }
}

// ------------------------------------------------------------------ sort (single CTA)
// pairs = T * K. counts / offsets in shared memory; rows of one expert are independent, so their
// order inside the expert's range is free. With align > 1 every *tile* starts at a multiple of `align`
// rows and holds at most tile_rows (<= align) pairs in its first rows (NVFP4 operands carry their scale
// factors in blocks of 128 rows, and a token tile must start on such a block): pair i of an expert sits at
// row off[e] + (i / tile_rows) * align + i % tile_rows. Every row of [0, row_cap) that holds no pair gets
// row_pair = -1 (nothing is gathered or computed for it); *total_rows is the end of the last tile's slot.
__global__ void __launch_bounds__(1024)
sort_kernel(const int* __restrict__ ids, int pairs, int expert_lo, int num_local, int tile_rows, int align, int row_cap,
            int* __restrict__ pair_row, int* __restrict__ row_pair, int* __restrict__ expert_off,
            int* __restrict__ tile_expert, int* __restrict__ tile_row0, int* __restrict__ tile_nrows,
            int max_tiles, int* __restrict__ total_rows) {
  extern __shared__ int sm_i[];
  int* cnt = sm_i;                       // [num_local]
  int* off = sm_i + num_local;           // [num_local + 1]
  const int tid = threadIdx.x, nt = blockDim.x;
  for (int e = tid; e < num_local; e += nt) cnt[e] = 0;
  __syncthreads();
  for (int i = tid; i < pairs; i += nt) {
    const int e = ids[i] - expert_lo;
    if (e >= 0 && e < num_local) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  // offsets and the tile work-list: thread e owns expert e (num_local <= blockDim.x = 1024); an exclusive block
  // scan over (rows, tiles) of the experts replaces a walk over the experts by one thread
  __shared__ int wsum[2][32];
  __shared__ int tot[2];
  {
    const int lane = tid & 31, warp = tid >> 5;
    const int c = tid < num_local ? cnt[tid] : 0;
    const int my_tiles = (c + tile_rows - 1) / tile_rows;
    const int my_rows = align > 1 ? my_tiles * align : c;
    int sr = my_rows, st = my_tiles;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int ur = __shfl_up_sync(0xffffffffu, sr, d), ut = __shfl_up_sync(0xffffffffu, st, d);
      if (lane >= d) { sr += ur; st += ut; }
    }
    if (lane == 31) { wsum[0][warp] = sr; wsum[1][warp] = st; }
    __syncthreads();
    if (warp == 0) {
      const int wr = wsum[0][lane], wt = wsum[1][lane];
      int ir = wr, it = wt;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int ur = __shfl_up_sync(0xffffffffu, ir, d), ut = __shfl_up_sync(0xffffffffu, it, d);
        if (lane >= d) { ir += ur; it += ut; }
      }
      wsum[0][lane] = ir - wr;                                   // rows / tiles in front of this warp
      wsum[1][lane] = it - wt;
      if (lane == 31) { tot[0] = ir; tot[1] = it; }
    }
    __syncthreads();
    const int row_base = wsum[0][warp] + sr - my_rows, tile_base = wsum[1][warp] + st - my_tiles;
    if (tid < num_local) {
      off[tid] = row_base;
      const int stride = align > 1 ? align : tile_rows;
      for (int j = 0; j < my_tiles && tile_base + j < max_tiles; ++j) {
        tile_expert[tile_base + j] = tid;
        tile_row0[tile_base + j] = row_base + j * stride;
        tile_nrows[tile_base + j] = min(tile_rows, c - j * tile_rows);
      }
    }
    if (tid == 0) { off[num_local] = tot[0]; *total_rows = tot[0]; }
    for (int i = tot[1] + tid; i < max_tiles; i += nt) { tile_expert[i] = -1; tile_row0[i] = 0; tile_nrows[i] = 0; }
    // rows that end up without a pair keep this -1 (the placement below overwrites the others)
    if (align > 1)
      for (int r = tid; r < row_cap; r += nt) row_pair[r] = -1;
  }
  __syncthreads();
  for (int e = tid; e <= num_local; e += nt) expert_off[e] = off[e];
  // placement: every thread takes pairs tid, tid + nt, ... and claims the next free row of its pair's
  // expert with a shared-memory counter. Which row of an expert a pair lands on therefore varies from
  // run to run, the result does not: a row's GEMM output is independent of its place in the tile and
  // the combine reads rows through pair_row in slot order.
  for (int e = tid; e < num_local; e += nt) cnt[e] = 0;         // reused as the running fill of each expert
  __syncthreads();
  for (int i = tid; i < pairs; i += nt) {
    const int e = ids[i] - expert_lo;
    if (e >= 0 && e < num_local) {
      const int k = atomicAdd(&cnt[e], 1);
      const int pos = off[e] + (align > 1 ? (k / tile_rows) * align + k % tile_rows : k);
      pair_row[i] = pos;
      row_pair[pos] = i;
    }
  }
  for (int i = tid; i < pairs; i += nt) {
    const int e = ids[i] - expert_lo;
    if (e < 0 || e >= num_local) pair_row[i] = -1;
  }
}

// ------------------------------------------------------------------ gather / combine
// dst row r = src row (row_pair[r] / K); 16-byte vectors; rows beyond *total_rows are skipped.
__global__ void gather_kernel(const uint8_t* __restrict__ src, long long src_ld, uint8_t* __restrict__ dst,
                              long long dst_ld, int row_bytes, const int* __restrict__ row_pair, int K,
                              const int* __restrict__ total_rows, int max_rows,
                              const float* __restrict__ src_scale, float* __restrict__ dst_scale,
                              int scale_groups, int src_scale_ld, int dst_scale_ld) {
  const int r = blockIdx.x;
  if (r >= *total_rows || r >= max_rows) return;
  const int pr = row_pair[r];
  uint4* d = reinterpret_cast<uint4*>(dst + (size_t)r * dst_ld);
  if (pr < 0) return;                             // padding up to the next expert's aligned first row
  const int tok = pr / K;
  const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)tok * src_ld);
  for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) d[i] = s[i];
  if (src_scale) {
    // scales stored [group][row]
    for (int gI = threadIdx.x; gI < scale_groups; gI += blockDim.x)
      dst_scale[(size_t)gI * dst_scale_ld + r] = src_scale[(size_t)gI * src_scale_ld + tok];
  }
}

// NVFP4 activations, one CTA per (token, slot) pair: the pair's sorted row takes the token's packed e2m1
// row, its per-token scale and its scale-factor bytes. The scale factors live in 512-byte tiles of 128 rows x
// 4 groups of 16 channels (the layout tcgen05.cp consumes); the four bytes of one row and one 64-channel
// group are one aligned word, moved from the token's tile to the sorted row's tile. Rows that hold no pair
// are left as they are: the GEMM computes their output columns from whatever they hold and stores none.
__global__ void gather_nvfp4_kernel(const uint8_t* __restrict__ src, long long src_ld, uint8_t* __restrict__ dst,
                                    long long dst_ld, int row_bytes, const int* __restrict__ pair_row, int K,
                                    int max_rows, const float* __restrict__ src_scale, float* __restrict__ dst_scale,
                                    const uint8_t* __restrict__ src_sf, uint8_t* __restrict__ dst_sf, int sf_k64) {
  const int r = pair_row[blockIdx.x];
  if (r < 0 || r >= max_rows) return;
  const int tok = blockIdx.x / K;
  const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)tok * src_ld);
  uint4* d = reinterpret_cast<uint4*>(dst + (size_t)r * dst_ld);
  for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) d[i] = s[i];
  if (threadIdx.x == 0) dst_scale[r] = src_scale[tok];
  const uint8_t* sfs = src_sf + (size_t)(tok >> 7) * sf_k64 * 512 + mb::sf_tile_offset(tok & 127, 0);
  uint8_t* sfd = dst_sf + (size_t)(r >> 7) * sf_k64 * 512 + mb::sf_tile_offset(r & 127, 0);
  for (int g = threadIdx.x; g < sf_k64; g += blockDim.x)
    *reinterpret_cast<uint32_t*>(sfd + (size_t)g * 512) = *reinterpret_cast<const uint32_t*>(sfs + (size_t)g * 512);
}

__global__ void combine_kernel(const float* __restrict__ y, long long y_ld, const int* __restrict__ pair_row,
                               const float* __restrict__ w, int K, int H, const float* __restrict__ addend,
                               float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16) {
  const int tok = blockIdx.x;
  // the hidden row is split over blockIdx.y: at decode sizes one CTA per token leaves most SMs idle
  for (int h = blockIdx.y * blockDim.x + threadIdx.x; h < H; h += gridDim.y * blockDim.x) {
    float acc = addend ? addend[(size_t)tok * H + h] : 0.f;
    for (int j = 0; j < K; ++j) {
      const int r = pair_row[(size_t)tok * K + j];
      if (r >= 0) acc += w[(size_t)tok * K + j] * y[(size_t)r * y_ld + h];
    }
    if (out_f32) out_f32[(size_t)tok * H + h] = acc;
    if (out_bf16) out_bf16[(size_t)tok * H + h] = __float2bfloat16(acc);
  }
}

// The whole tail of a MoE block in one pass over the token's hidden row:
//   out = bf16( residual + sum_j w_j y[pair_row_j] + sigmoid(gate_logit) * shared )
// (shared expert, its sigmoid gate and the residual are each optional).
__global__ void moe_finish_kernel(const float* __restrict__ y, long long y_ld, const int* __restrict__ pair_row,
                                  const float* __restrict__ w, int K, int H,
                                  const __nv_bfloat16* __restrict__ shared, long long shared_ld,
                                  const float* __restrict__ gate_logit, long long gate_ld,
                                  const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out) {
  const int tok = blockIdx.x;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  float sg = 1.f;
  if (gate_logit) sg = 1.f / (1.f + __expf(-gate_logit[(size_t)tok * gate_ld]));
  int rows[32];
  float ws[32];
  for (int j = 0; j < K; ++j) {
    rows[j] = pair_row[(size_t)tok * K + j];
    ws[j] = w[(size_t)tok * K + j];
  }
  for (int h = (blockIdx.y * blockDim.x + threadIdx.x) * 2; h < H; h += gridDim.y * blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    for (int j = 0; j < K; ++j) {
      if (rows[j] >= 0) {
        const float2 v = *reinterpret_cast<const float2*>(y + (size_t)rows[j] * y_ld + h);
        a0 += ws[j] * v.x;
        a1 += ws[j] * v.y;
      }
    }
    if (shared) {
      const float2 sv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(shared + (size_t)tok * shared_ld + h));
      a0 += sg * sv.x;
      a1 += sg * sv.y;
    }
    if (residual) {
      const float2 rv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(residual + (size_t)tok * H + h));
      a0 += rv.x;
      a1 += rv.y;
    }
    *reinterpret_cast<__nv_bfloat162*>(out + (size_t)tok * H + h) = __floats2bfloat162_rn(a0, a1);
  }
}

}  // namespace

extern "C" {

int mb_moe_finish(const float* y, long long y_ld, const int* pair_row, const float* w, int T, int K, int H,
                  const void* shared, long long shared_ld, const float* gate_logit, long long gate_ld,
                  const void* residual, void* out, cudaStream_t stream) {
  if (!y || !pair_row || !w || !out || T <= 0 || K <= 0 || K > 32 || H % 2 || y_ld % 2 || shared_ld % 2)
    return MB_ERR_BAD_ARG;
  const int gy = T >= 2048 ? 1 : min(8, (H + 511) / 512);
  return (int)mb::launch_kernel(moe_finish_kernel, dim3(T, gy), dim3(256), 0, stream, y, y_ld, pair_row, w, K, H,
                                reinterpret_cast<const __nv_bfloat16*>(shared), shared_ld, gate_logit, gate_ld,
                                reinterpret_cast<const __nv_bfloat16*>(residual),
                                reinterpret_cast<__nv_bfloat16*>(out));
}

int mb_moe_route(const float* logits, long long ld, int T, int E, int K, int mode, const float* bias,
                 int n_group, int topk_group, int renorm, float scaling, float* out_w, int* out_id,
                 cudaStream_t stream) {
  if (!logits || !out_w || !out_id || T <= 0 || E <= 0 || E > 512 || K <= 0 || K > 32 || K > E)
    return MB_ERR_BAD_ARG;
  if (n_group > 1 && (E % n_group || n_group > 32 || topk_group > n_group)) return MB_ERR_BAD_ARG;
  route_kernel<<<(T + 3) / 4, 128, 0, stream>>>(logits, ld, T, E, K, mode, bias, n_group, topk_group,
                                               renorm, scaling, out_w, out_id, K, -1, -1);
  return (int)cudaGetLastError();
}

// As mb_moe_route, with the outputs [T, K + 1]: slot K of every token is expert `shared_id` with
// weight sigmoid(logits[gate_col]) (or 1 when gate_col < 0). Top-k runs over the first E columns.
int mb_moe_route_shared(const float* logits, long long ld, int T, int E, int K, int mode, const float* bias,
                        int n_group, int topk_group, int renorm, float scaling, float* out_w, int* out_id,
                        int shared_id, int gate_col, cudaStream_t stream) {
  if (!logits || !out_w || !out_id || T <= 0 || E <= 0 || E > 512 || K <= 0 || K >= 32 || K > E || shared_id < 0)
    return MB_ERR_BAD_ARG;
  if (n_group > 1 && (E % n_group || n_group > 32 || topk_group > n_group)) return MB_ERR_BAD_ARG;
  route_kernel<<<(T + 3) / 4, 128, 0, stream>>>(logits, ld, T, E, K, mode, bias, n_group, topk_group,
                                               renorm, scaling, out_w, out_id, K + 1, shared_id, gate_col);
  return (int)cudaGetLastError();
}

// `align` > 1: every tile starts at a multiple of `align` rows; row_pair has `row_cap` entries
// (>= max_tiles * align covers every routing); tile_rows must divide `align`.
int mb_moe_sort_aligned(const int* ids, int pairs, int expert_lo, int num_local, int tile_rows, int align, int row_cap,
                        int* pair_row, int* row_pair, int* expert_off, int* tile_expert, int* tile_row0,
                        int* tile_nrows, int max_tiles, int* total_rows, cudaStream_t stream) {
  if (!ids || pairs <= 0 || num_local <= 0 || num_local > 1024 || tile_rows <= 0 || align <= 0 || (align > 1 && (align % tile_rows || row_cap < pairs)))
    return MB_ERR_BAD_ARG;
  const size_t smem = (2 * (size_t)num_local + 1) * sizeof(int);
  sort_kernel<<<1, 1024, smem, stream>>>(ids, pairs, expert_lo, num_local, tile_rows, align, row_cap, pair_row, row_pair,
                                         expert_off, tile_expert, tile_row0, tile_nrows, max_tiles, total_rows);
  return (int)cudaGetLastError();
}

int mb_moe_sort(const int* ids, int pairs, int expert_lo, int num_local, int tile_rows, int* pair_row,
                int* row_pair, int* expert_off, int* tile_expert, int* tile_row0, int* tile_nrows,
                int max_tiles, int* total_rows, cudaStream_t stream) {
  return mb_moe_sort_aligned(ids, pairs, expert_lo, num_local, tile_rows, 1, pairs, pair_row, row_pair, expert_off,
                             tile_expert, tile_row0, tile_nrows, max_tiles, total_rows, stream);
}

int mb_moe_gather(const void* src, long long src_ld, void* dst, long long dst_ld, int row_bytes,
                  const int* row_pair, int K, const int* total_rows, int max_rows, const float* src_scale,
                  float* dst_scale, int scale_groups, int src_scale_ld, int dst_scale_ld,
                  cudaStream_t stream) {
  if (!src || !dst || row_bytes % 16 || max_rows <= 0) return MB_ERR_BAD_ARG;
  gather_kernel<<<max_rows, 128, 0, stream>>>(reinterpret_cast<const uint8_t*>(src), src_ld,
                                              reinterpret_cast<uint8_t*>(dst), dst_ld, row_bytes, row_pair, K,
                                              total_rows, max_rows, src_scale, dst_scale, scale_groups,
                                              src_scale_ld, dst_scale_ld);
  return (int)cudaGetLastError();
}

int mb_moe_gather_nvfp4(const void* src, long long src_ld, void* dst, long long dst_ld, int row_bytes,
                        const int* pair_row, int pairs, int K, int max_rows, const float* src_scale,
                        float* dst_scale, const void* src_sf, void* dst_sf, int sf_k64, cudaStream_t stream) {
  if (!src || !dst || !pair_row || !src_scale || !dst_scale || !src_sf || !dst_sf || sf_k64 <= 0 || row_bytes % 16 ||
      pairs <= 0 || K <= 0 || max_rows <= 0)
    return MB_ERR_BAD_ARG;
  gather_nvfp4_kernel<<<pairs, 64, 0, stream>>>(reinterpret_cast<const uint8_t*>(src), src_ld,
                                                reinterpret_cast<uint8_t*>(dst), dst_ld, row_bytes, pair_row, K,
                                                max_rows, src_scale, dst_scale,
                                                reinterpret_cast<const uint8_t*>(src_sf),
                                                reinterpret_cast<uint8_t*>(dst_sf), sf_k64);
  return (int)cudaGetLastError();
}

int mb_moe_combine(const float* y, long long y_ld, const int* pair_row, const float* w, int T, int K, int H,
                   const float* addend, float* out_f32, void* out_bf16, cudaStream_t stream) {
  if (!y || !pair_row || !w || T <= 0) return MB_ERR_BAD_ARG;
  const int gy = T >= 2048 ? 1 : min(8, (H + 255) / 256);
  combine_kernel<<<dim3(T, gy), 256, 0, stream>>>(y, y_ld, pair_row, w, K, H, addend, out_f32,
                                        reinterpret_cast<__nv_bfloat16*>(out_bf16));
  return (int)cudaGetLastError();
}

}  // extern "C"
