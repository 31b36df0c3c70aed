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
#include <cstdlib>

namespace {

constexpr int kKeysPerCta = 128;     // two keys per thread, four threads per key

// Four threads share a key: each keeps a quarter of the key's channels in registers as fp32 and walks all
// indexer heads, reading the matching quarter of the head's query from shared memory (fp32, rows padded so
// that the four quarters fall on different banks); the four partial dot products meet through two shuffles
// before the ReLU. Per (key, head) that is DI / 4 FMAs per thread and nothing else in the inner loop.
template <int DI>
__global__ void __launch_bounds__(256)
index_score_kernel(const __nv_bfloat16* __restrict__ iq, const float* __restrict__ iw,
                   const __nv_bfloat16* __restrict__ kc, const int* __restrict__ block_table, int max_blocks,
                   const int* __restrict__ row_seq, const int* __restrict__ row_ctx, float* __restrict__ scores,
                   long long ld, int Hi, int block_size, long long num_blocks, uint32_t* status) {
  constexpr int Q = DI / 4;                 // channels per thread
  constexpr int QS = Q + 4;                 // padded quarter: quarter p starts at bank 4p
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* qs = reinterpret_cast<float*>(smem_raw);                                      // [Hi][4][QS]
  float* ws = qs + (size_t)Hi * 4 * QS;                                                // [Hi]
  const int t = blockIdx.y, s0 = blockIdx.x * kKeysPerCta;
  const int ctx = row_ctx[t];
  const int part = threadIdx.x & 3;
  const int pos0 = s0 + (threadIdx.x >> 2), pos1 = pos0 + kKeysPerCta / 2;
  if (s0 >= ctx) {                                          // the whole tile is past this row's context
    if (part == 0) {
      if (pos0 < ld) scores[(size_t)t * ld + pos0] = -INFINITY;
      if (pos1 < ld) scores[(size_t)t * ld + pos1] = -INFINITY;
    }
    return;
  }
  const __nv_bfloat16* q = iq + (size_t)t * Hi * DI;
  for (int i = threadIdx.x; i < Hi * DI; i += blockDim.x) {
    const int h = i / DI, d = i - h * DI;
    qs[((size_t)h * 4 + d / Q) * QS + d % Q] = __bfloat162float(q[i]);
  }
  for (int i = threadIdx.x; i < Hi; i += blockDim.x) ws[i] = iw[(size_t)t * Hi + i];
  __syncthreads();
  float k[2][Q];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int pos = u ? pos1 : pos0;
#pragma unroll
    for (int i = 0; i < Q; ++i) k[u][i] = 0.f;
    if (pos < ctx) {
      const int blk = block_table[(size_t)row_seq[t] * max_blocks + pos / block_size];
      if (blk < 0 || blk >= num_blocks) {
        if (status) atomicCAS(status, 0u, MB_ST_BOUNDS);
      } else {
        const uint4* kr = reinterpret_cast<const uint4*>(kc + ((size_t)blk * block_size + pos % block_size) * DI + part * Q);
#pragma unroll
        for (int i = 0; i < Q / 8; ++i) {
          const uint4 v = kr[i];
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h2[j]);
            k[u][8 * i + 2 * j] = f.x;
            k[u][8 * i + 2 * j + 1] = f.y;
          }
        }
      }
    }
  }
  float acc0 = 0.f, acc1 = 0.f;
  for (int h = 0; h < Hi; ++h) {
    const float4* qh = reinterpret_cast<const float4*>(qs + ((size_t)h * 4 + part) * QS);
    float d0 = 0.f, d1 = 0.f;
#pragma unroll
    for (int i = 0; i < Q / 4; ++i) {
      const float4 a = qh[i];                     // one shared-memory read feeds both keys
      d0 = fmaf(a.x, k[0][4 * i], d0);
      d1 = fmaf(a.x, k[1][4 * i], d1);
      d0 = fmaf(a.y, k[0][4 * i + 1], d0);
      d1 = fmaf(a.y, k[1][4 * i + 1], d1);
      d0 = fmaf(a.z, k[0][4 * i + 2], d0);
      d1 = fmaf(a.z, k[1][4 * i + 2], d1);
      d0 = fmaf(a.w, k[0][4 * i + 3], d0);
      d1 = fmaf(a.w, k[1][4 * i + 3], d1);
    }
    d0 += __shfl_xor_sync(0xffffffffu, d0, 1);
    d1 += __shfl_xor_sync(0xffffffffu, d1, 1);
    d0 += __shfl_xor_sync(0xffffffffu, d0, 2);
    d1 += __shfl_xor_sync(0xffffffffu, d1, 2);
    const float w = ws[h];
    acc0 = fmaf(w, fmaxf(d0, 0.f), acc0);
    acc1 = fmaf(w, fmaxf(d1, 0.f), acc1);
  }
  if (part == 0) {
    if (pos0 < ld) scores[(size_t)t * ld + pos0] = pos0 < ctx ? acc0 : -INFINITY;
    if (pos1 < ld) scores[(size_t)t * ld + pos1] = pos1 < ctx ? acc1 : -INFINITY;
  }
}

// Tensor-core form for the common indexer shape (a multiple of 16 heads, up to 64; 128 channels): the score is
// a [heads x 128] by [128 x keys] product followed by ReLU, the head weights and a sum over heads. One warp keeps
// the whole query as m16n8k16 A fragments in registers (loaded once, straight from global memory) and walks
// tiles of eight keys; the B fragments are the keys' own rows, read from the paged cache as 32-bit pairs in the
// fragment layout (lane = (key, channel pair)), so nothing is staged in shared memory. The epilogue applies
// ReLU and the head weights on the accumulators and reduces over heads with three shuffles.
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kTcWarps = 4;          // keys per CTA = 4 warps x tiles per warp (launcher's choice) x 8

template <int MT>                                          // MT head tiles of 16
__global__ void __launch_bounds__(kTcWarps * 32)
index_score_tc_kernel(const __nv_bfloat16* __restrict__ iq, const float* __restrict__ iw,
                      const __nv_bfloat16* __restrict__ kc, const int* __restrict__ block_table, int max_blocks,
                      const int* __restrict__ row_seq, const int* __restrict__ row_ctx, float* __restrict__ scores,
                      long long ld, int block_size, long long num_blocks, int tiles_per_warp, uint32_t* status) {
  constexpr int DI = 128, KS = DI / 16, Hi = MT * 16;
  const int t = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, c = lane & 3;
  const int ctx = row_ctx[t];
  const int key0 = (blockIdx.x * kTcWarps + warp) * tiles_per_warp * 8;
  if (key0 >= ld) return;
  if (key0 >= ctx) {                                         // nothing of this warp's span is visible
    for (int i = lane; i < tiles_per_warp * 8; i += 32)
      if (key0 + i < ld) scores[(size_t)t * ld + key0 + i] = -INFINITY;
    return;
  }
  // A fragments of the whole query: a[mt][ks] = rows (mt*16 + r, + 8), channel pairs (ks*16 + 2c, + 8)
  uint32_t a[MT][KS][4];
  const uint32_t* q32 = reinterpret_cast<const uint32_t*>(iq + (size_t)t * Hi * DI);
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int row = mt * 16 + r, col = ks * 16 + 2 * c;
      a[mt][ks][0] = q32[(row * DI + col) >> 1];
      a[mt][ks][1] = q32[((row + 8) * DI + col) >> 1];
      a[mt][ks][2] = q32[(row * DI + col + 8) >> 1];
      a[mt][ks][3] = q32[((row + 8) * DI + col + 8) >> 1];
    }
  float w_lo[MT], w_hi[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    w_lo[mt] = iw[(size_t)t * Hi + mt * 16 + r];
    w_hi[mt] = iw[(size_t)t * Hi + mt * 16 + r + 8];
  }
  const int seq = row_seq[t];
  for (int nt = 0; nt < tiles_per_warp; ++nt) {
    const int base = key0 + nt * 8;
    if (base >= ld) break;
    const int pos = base + r;                                // this lane's key (the fragment's column)
    const uint32_t* krow = nullptr;
    if (pos < ctx) {
      const int blk = block_table[(size_t)seq * max_blocks + pos / block_size];
      if (blk < 0 || blk >= num_blocks) {
        if (status) atomicCAS(status, 0u, MB_ST_BOUNDS);
      } else {
        krow = reinterpret_cast<const uint32_t*>(kc + ((size_t)blk * block_size + pos % block_size) * DI);
      }
    }
    uint32_t b[KS][2];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      b[ks][0] = krow ? krow[(ks * 16 + 2 * c) >> 1] : 0u;
      b[ks][1] = krow ? krow[(ks * 16 + 2 * c + 8) >> 1] : 0u;
    }
    float s0 = 0.f, s1 = 0.f;                                // keys base + 2c and base + 2c + 1, this lane's head rows
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) mma_bf16_16816(acc, a[mt][ks], b[ks][0], b[ks][1]);
      s0 += w_lo[mt] * fmaxf(acc[0], 0.f) + w_hi[mt] * fmaxf(acc[2], 0.f);
      s1 += w_lo[mt] * fmaxf(acc[1], 0.f) + w_hi[mt] * fmaxf(acc[3], 0.f);
    }
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {                 // over the eight head rows a lane group holds
      s0 += __shfl_xor_sync(0xffffffffu, s0, off);
      s1 += __shfl_xor_sync(0xffffffffu, s1, off);
    }
    if (r == 0) {
      const int p0 = base + 2 * c, p1 = p0 + 1;
      if (p0 < ld) scores[(size_t)t * ld + p0] = p0 < ctx ? s0 : -INFINITY;
      if (p1 < ld) scores[(size_t)t * ld + p1] = p1 < ctx ? s1 : -INFINITY;
    }
  }
}

// order-preserving map float -> uint32 (larger float = larger integer)
__device__ __forceinline__ uint32_t f2key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// exclusive prefix of `v` over the block (1024 threads), and the block total
__device__ __forceinline__ int block_excl_scan(int v, int* warp_tot, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, inc, off);
    if (lane >= off) inc += n;
  }
  __syncthreads();                                          // warp_tot is free again
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  int before = 0, tot = 0;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
    const int c = warp_tot[w];
    if (w < warp) before += c;
    tot += c;
  }
  total = tot;
  return before + inc - v;
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
  // the number of entries equal to it that still belong to the selection. Lanes that hit the same
  // bin are counted by one atomic (scores cluster on few exponents, so the first pass would
  // otherwise serialise on a handful of counters).
  uint32_t prefix = 0, mask = 0;
  int need = k;
  const int n_up = (n + 31) / 32 * 32;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_up; i += blockDim.x) {
      const uint32_t key = i < n ? f2key(sc[i]) : 0u;
      const bool in = i < n && (key & mask) == prefix;
      const unsigned part = __ballot_sync(0xffffffffu, in);
      if (in) {
        const int bin = (key >> shift) & 255;
        const unsigned peers = __match_any_sync(part, bin);
        if ((int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], __popc(peers));
      }
    }
    __syncthreads();
    {
      // bins in descending order: thread i looks at bin 255 - i; the entries above it are the exclusive
      // prefix, and the bin that takes the count across `need` holds the k-th largest key
      const int b = 255 - (int)threadIdx.x;
      const int c = threadIdx.x < 256 ? hist[b] : 0;
      int tot;
      const int above = block_excl_scan(c, warp_tot, tot);
      if (threadIdx.x < 256 && above < need && need <= above + c) {
        s_prefix = prefix | ((uint32_t)b << shift);
        s_need = need - above;
      }
    }
    __syncthreads();
    prefix = s_prefix;
    need = s_need;
    mask |= 255u << shift;
    __syncthreads();
  }
  // ordered compaction: warp w owns the contiguous segment [w * seg, (w + 1) * seg) and walks it 32 entries
  // at a time (coalesced); a counting pass gives every warp its base in the output and the number of
  // threshold-equal entries before it, a second pass places the selected entries with ballots
  __shared__ int gt_w[32], eq_w[32], base_w[32], eqb_w[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int seg = ((n + 31) / 32 + 31) / 32 * 32;
  const int lo = warp * seg, hi = min(n, lo + seg);
  int gt = 0, eq = 0;
  for (int c0 = lo; c0 < hi; c0 += 32) {
    const int i = c0 + lane;
    const uint32_t key = i < hi ? f2key(sc[i]) : 0u;
    gt += __popc(__ballot_sync(0xffffffffu, i < hi && key > prefix));
    eq += __popc(__ballot_sync(0xffffffffu, i < hi && key == prefix));
  }
  if (lane == 0) {
    gt_w[warp] = gt;
    eq_w[warp] = eq;
  }
  __syncthreads();
  if (warp == 0) {
    const int g = gt_w[lane], e = eq_w[lane];
    int inc = e;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, inc, off);
      if (lane >= off) inc += v;
    }
    const int eq_before = inc - e;
    const int sel = g + max(0, min(e, need - eq_before));
    int inc2 = sel;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, inc2, off);
      if (lane >= off) inc2 += v;
    }
    base_w[lane] = inc2 - sel;
    eqb_w[lane] = eq_before;
  }
  __syncthreads();
  int p = base_w[warp], eq_run = eqb_w[warp];
  const unsigned lt = (1u << lane) - 1u;
  for (int c0 = lo; c0 < hi; c0 += 32) {
    const int i = c0 + lane;
    const uint32_t key = i < hi ? f2key(sc[i]) : 0u;
    const bool is_eq = i < hi && key == prefix;
    const unsigned eqm = __ballot_sync(0xffffffffu, is_eq);
    const bool sel = (i < hi && key > prefix) || (is_eq && eq_run + __popc(eqm & lt) < need);
    const unsigned sm = __ballot_sync(0xffffffffu, sel);
    const int at = p + __popc(sm & lt);
    if (sel && at < k) out[at] = i;
    p += __popc(sm);
    eq_run += __popc(eqm);
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

static bool tc_off() {
  static const bool off = [] {
    const char* e = getenv("METRALE_INDEX_TC");
    return e && e[0] == '0';
  }();
  return off;
}

extern "C" int mb_index_score(const void* iq, const void* iw, const void* kc, const void* block_table, int max_blocks,
                              const void* row_seq, const void* row_ctx, void* scores, long long ld, int T, int Hi,
                              int Di, int block_size, long long num_blocks, void* status, cudaStream_t stream) {
  if (!iq || !iw || !kc || !scores || T <= 0 || Hi <= 0 || Hi > 128 || ld <= 0) return MB_ERR_BAD_ARG;
  const dim3 grid((unsigned)((ld + kKeysPerCta - 1) / kKeysPerCta), T);
  const size_t smem = (size_t)Hi * 4 * (Di / 4 + 4) * 4 + (size_t)Hi * 4;
  if (smem > 200 * 1024 || Di % 32) return MB_ERR_TOO_LARGE;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(index_score_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(index_score_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
#define MB_IDX_LAUNCH(DI)                                                                                        \
  index_score_kernel<DI><<<grid, 256, smem, stream>>>(                                                           \
      static_cast<const __nv_bfloat16*>(iq), static_cast<const float*>(iw), static_cast<const __nv_bfloat16*>(kc), \
      static_cast<const int*>(block_table), max_blocks, static_cast<const int*>(row_seq),                        \
      static_cast<const int*>(row_ctx), static_cast<float*>(scores), ld, Hi, block_size, num_blocks,             \
      static_cast<uint32_t*>(status))
  if (Di == 128 && Hi % 16 == 0 && Hi <= 64 && !(tc_off())) {
    // 16 key tiles per warp amortise the query fragments best; fewer when that would leave SMs idle
    int tpw = 16;
    while (tpw > 2 && (long long)T * ((ld + kTcWarps * tpw * 8 - 1) / (kTcWarps * tpw * 8)) < 2 * 148) tpw >>= 1;
    const dim3 g2((unsigned)((ld + kTcWarps * tpw * 8 - 1) / (kTcWarps * tpw * 8)), T);
#define MB_IDX_TC(MT)                                                                                              \
  index_score_tc_kernel<MT><<<g2, kTcWarps * 32, 0, stream>>>(                                                     \
      static_cast<const __nv_bfloat16*>(iq), static_cast<const float*>(iw), static_cast<const __nv_bfloat16*>(kc), \
      static_cast<const int*>(block_table), max_blocks, static_cast<const int*>(row_seq),                          \
      static_cast<const int*>(row_ctx), static_cast<float*>(scores), ld, block_size, num_blocks, tpw,              \
      static_cast<uint32_t*>(status))
    switch (Hi / 16) {
      case 1: MB_IDX_TC(1); break;
      case 2: MB_IDX_TC(2); break;
      case 3: MB_IDX_TC(3); break;
      default: MB_IDX_TC(4); break;
    }
#undef MB_IDX_TC
    return (int)cudaGetLastError();
  }
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
