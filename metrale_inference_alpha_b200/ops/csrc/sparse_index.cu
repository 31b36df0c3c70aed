// Sparse (indexed) attention: a light indexer scores every cached token for every query row, the k
// best tokens per row are selected, and attention runs over those tokens only.
//
//   index_score   score[t, s] = sum_h w[t, h] * relu(<q_idx[t, h, :], k_idx[s, :]>)   for s < ctx[t]
//                 (one small head-shared key per token, cached beside the KV rows; -inf past ctx[t])
//   topk_select   per row: the k largest scores, ties to the lower position, returned in ascending
//                 position order (so the result does not depend on thread timing); rows with
//                 ctx <= k select everything. Radix select over the order-preserving integer image of
//                 the scores (4 passes of 8 bits), then an ordered compaction.
//   gather_rows   the selected tokens' cache rows, through the block table, into a compact per-row
//                 paged buffer that the dense attention kernel reads with an identity block table.
//
// Reference behaviour covered: kernels/gb10/common/dsa_indexer.cu (score, deterministic top-k,
// selection expansion, compaction) and the sparse decode of glm5next_dsa_mla_decode.cu; there the
// candidates are pools of tokens, here single tokens (the DeepSeek sparse-attention form).
#include "common.cuh"

namespace {

constexpr int kKeysPerCta = 64;

template <int DI>
__global__ void __launch_bounds__(256)
index_score_kernel(const __nv_bfloat16* __restrict__ iq, const float* __restrict__ iw,
                   const __nv_bfloat16* __restrict__ kc, const int* __restrict__ block_table, int max_blocks,
                   const int* __restrict__ row_seq, const int* __restrict__ row_ctx, float* __restrict__ scores,
                   long long ld, int Hi, int block_size, long long num_blocks, uint32_t* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat162* qs = reinterpret_cast<__nv_bfloat162*>(smem_raw);                  // [Hi][DI / 2]
  float* ws = reinterpret_cast<float*>(smem_raw + (size_t)Hi * DI * 2);               // [Hi]
  const int t = blockIdx.y, s0 = blockIdx.x * kKeysPerCta;
  const int ctx = row_ctx[t];
  const int key = threadIdx.x >> 2, hg = threadIdx.x & 3;
  const int pos = s0 + key;
  if (s0 >= ctx) {                                          // the whole tile is past this row's context
    if (hg == 0 && pos < ld) scores[(size_t)t * ld + pos] = -INFINITY;
    return;
  }
  const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(iq + (size_t)t * Hi * DI);
  for (int i = threadIdx.x; i < Hi * DI / 2; i += blockDim.x) qs[i] = q2[i];
  for (int i = threadIdx.x; i < Hi; i += blockDim.x) ws[i] = iw[(size_t)t * Hi + i];
  __syncthreads();
  float acc = 0.f;
  if (pos < ctx) {
    const int blk = block_table[(size_t)row_seq[t] * max_blocks + pos / block_size];
    if (blk < 0 || blk >= num_blocks) {
      if (status) atomicCAS(status, 0u, MB_ST_BOUNDS);
    } else {
      const uint4* kr = reinterpret_cast<const uint4*>(kc + ((size_t)blk * block_size + pos % block_size) * DI);
      __nv_bfloat162 k2[DI / 2];
#pragma unroll
      for (int i = 0; i < DI / 8; ++i) *reinterpret_cast<uint4*>(&k2[4 * i]) = kr[i];
      for (int h = hg; h < Hi; h += 4) {
        const __nv_bfloat162* qh = qs + (size_t)h * (DI / 2);
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < DI / 2; ++i) {
          const float2 a = __bfloat1622float2(qh[i]), b = __bfloat1622float2(k2[i]);
          dot = fmaf(a.x, b.x, dot);
          dot = fmaf(a.y, b.y, dot);
        }
        acc = fmaf(ws[h], fmaxf(dot, 0.f), acc);
      }
    }
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  if (hg == 0 && pos < ld) scores[(size_t)t * ld + pos] = pos < ctx ? acc : -INFINITY;
}

// order-preserving map float -> uint32 (larger float = larger integer)
__device__ __forceinline__ uint32_t f2key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// exclusive prefix of `flag` over the block (1024 threads), and the block total
__device__ __forceinline__ int block_excl_scan(int flag, int* warp_tot, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned m = __ballot_sync(0xffffffffu, flag);
  const int in_warp = __popc(m & ((1u << lane) - 1u));
  __syncthreads();                                          // warp_tot is free again
  if (lane == 0) warp_tot[warp] = __popc(m);
  __syncthreads();
  int before = 0, tot = 0;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
    const int c = warp_tot[w];
    if (w < warp) before += c;
    tot += c;
  }
  total = tot;
  return before + in_warp;
}

__global__ void __launch_bounds__(1024)
topk_select_kernel(const float* __restrict__ scores, long long ld, const int* __restrict__ row_ctx, int k,
                   int* __restrict__ idx, int* __restrict__ count) {
  __shared__ int hist[256];
  __shared__ int warp_tot[32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  const int t = blockIdx.x;
  const int n = row_ctx[t];
  const float* sc = scores + (size_t)t * ld;
  int* out = idx + (size_t)t * k;
  if (n <= k) {
    for (int i = threadIdx.x; i < k; i += blockDim.x) out[i] = i < n ? i : -1;
    if (threadIdx.x == 0) count[t] = n < 0 ? 0 : n;
    return;
  }
  // radix select: after the four passes `prefix` is the key of the k-th largest score and `need`
  // the number of entries equal to it that still belong to the selection
  uint32_t prefix = 0, mask = 0;
  int need = k;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t key = f2key(sc[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int rem = need, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= rem) break;
        rem -= hist[b];
      }
      s_prefix = prefix | ((uint32_t)b << shift);
      s_need = rem;
    }
    __syncthreads();
    prefix = s_prefix;
    need = s_need;
    mask |= 255u << shift;
    __syncthreads();
  }
  // ordered compaction: everything above the threshold, and the first `need` entries equal to it
  int base = 0, eq_seen = 0;
  for (int c0 = 0; c0 < n; c0 += blockDim.x) {
    const int i = c0 + threadIdx.x;
    const uint32_t key = i < n ? f2key(sc[i]) : 0u;
    const int gt = i < n && key > prefix, eq = i < n && key == prefix;
    int eq_tot, sel_tot;
    const int eq_rank = eq_seen + block_excl_scan(eq, warp_tot, eq_tot);
    const int sel = gt || (eq && eq_rank < need);
    const int p = base + block_excl_scan(sel, warp_tot, sel_tot);
    if (sel && p < k) out[p] = i;
    base += sel_tot;
    eq_seen += eq_tot;
  }
  if (threadIdx.x == 0) count[t] = k;
}

// one warp per selected token: 16-byte copies of one cache row
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ cache, const int* __restrict__ block_table, int max_blocks,
                   const int* __restrict__ row_seq, const int* __restrict__ idx, const int* __restrict__ count,
                   uint4* __restrict__ dst, int k, int k_pad, int row_u4, int block_size, long long num_blocks,
                   long long total, uint32_t* status) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= total) return;
  const int t = (int)(w / k), j = (int)(w - (long long)t * k);
  if (j >= count[t]) return;
  const int tok = idx[(size_t)t * k + j];
  if (tok < 0) return;
  const int blk = block_table[(size_t)row_seq[t] * max_blocks + tok / block_size];
  if (blk < 0 || blk >= num_blocks) {
    if (status && (threadIdx.x & 31) == 0) atomicCAS(status, 0u, MB_ST_BOUNDS);
    return;
  }
  const uint4* src = cache + ((size_t)blk * block_size + tok % block_size) * row_u4;
  uint4* d = dst + ((size_t)t * k_pad + j) * row_u4;
  for (int i = threadIdx.x & 31; i < row_u4; i += 32) d[i] = src[i];
}

}  // namespace

extern "C" int mb_index_score(const void* iq, const void* iw, const void* kc, const void* block_table, int max_blocks,
                              const void* row_seq, const void* row_ctx, void* scores, long long ld, int T, int Hi,
                              int Di, int block_size, long long num_blocks, void* status, cudaStream_t stream) {
  if (!iq || !iw || !kc || !scores || T <= 0 || Hi <= 0 || Hi > 128 || ld <= 0) return MB_ERR_BAD_ARG;
  const dim3 grid((unsigned)((ld + kKeysPerCta - 1) / kKeysPerCta), T);
  const size_t smem = (size_t)Hi * Di * 2 + (size_t)Hi * 4;
  if (smem > 48 * 1024) return MB_ERR_TOO_LARGE;
#define MB_IDX_LAUNCH(DI)                                                                                        \
  index_score_kernel<DI><<<grid, 256, smem, stream>>>(                                                           \
      static_cast<const __nv_bfloat16*>(iq), static_cast<const float*>(iw), static_cast<const __nv_bfloat16*>(kc), \
      static_cast<const int*>(block_table), max_blocks, static_cast<const int*>(row_seq),                        \
      static_cast<const int*>(row_ctx), static_cast<float*>(scores), ld, Hi, block_size, num_blocks,             \
      static_cast<uint32_t*>(status))
  if (Di == 128) MB_IDX_LAUNCH(128);
  else if (Di == 64) MB_IDX_LAUNCH(64);
  else return MB_ERR_UNSUPPORTED;
#undef MB_IDX_LAUNCH
  return (int)cudaGetLastError();
}

extern "C" int mb_topk_select(const void* scores, long long ld, const void* row_ctx, int T, int k, void* idx,
                              void* count, cudaStream_t stream) {
  if (!scores || !row_ctx || !idx || !count || T <= 0 || k <= 0) return MB_ERR_BAD_ARG;
  topk_select_kernel<<<T, 1024, 0, stream>>>(static_cast<const float*>(scores), ld, static_cast<const int*>(row_ctx),
                                             k, static_cast<int*>(idx), static_cast<int*>(count));
  return (int)cudaGetLastError();
}

extern "C" int mb_gather_rows(const void* cache, const void* block_table, int max_blocks, const void* row_seq,
                              const void* idx, const void* count, void* dst, int T, int k, int k_pad, int row_bytes,
                              int block_size, long long num_blocks, void* status, cudaStream_t stream) {
  if (!cache || !idx || !dst || T <= 0 || k <= 0 || k_pad < k || row_bytes % 16) return MB_ERR_BAD_ARG;
  const long long total = (long long)T * k;
  const long long ctas = (total + 7) / 8;
  gather_rows_kernel<<<(unsigned)ctas, 256, 0, stream>>>(
      static_cast<const uint4*>(cache), static_cast<const int*>(block_table), max_blocks,
      static_cast<const int*>(row_seq), static_cast<const int*>(idx), static_cast<const int*>(count),
      static_cast<uint4*>(dst), k, k_pad, row_bytes / 16, block_size, num_blocks, total,
      static_cast<uint32_t*>(status));
  return (int)cudaGetLastError();
}
