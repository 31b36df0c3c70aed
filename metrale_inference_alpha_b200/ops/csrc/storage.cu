// Kernels of the KV storage tier: a sequence whose KV blocks live in files is attended one tile of
// blocks at a time as the tiles arrive in a small device scratch pool, and a low-rank predictor ranks
// blocks by importance so the tier knows which ones to keep close.
//
//   lowrank_project   rows [R, D] (bf16 queries, or K rows of paged blocks in bf16 / e4m3) times a
//                     fixed projection P [D, r] -> bf16 [.., r]
//   predictor_score   score[seq, b] = max over (query head, token of block b) of
//                     <q_lr[head], K_lr[block, head / G, token]>
//   kv_tile_attn      folds one tile of blocks into the running online-softmax state (m, l, o) of
//                     every (sequence, query head); one CTA per (sequence, kv head) so that the G query
//                     heads of a group share each K / V row, one warp per token, the lanes across the
//                     head dimension with 8- or 16-byte loads; optionally writes o / l on the last tile
//   attn_finalize     o / l as bf16 (0 where nothing was attended)
//
// The tile kernel is a streaming CUDA-core kernel on purpose: its input arrives from NVMe / host
// memory at tens of GB/s, two orders of magnitude below what the 16-row mma.sync decode kernel
// needs to be worth its fixed cost.
//
// Reference behaviour covered: crates/storage/kernels/{q_lowrank_project,kv_lowrank_project,
// predictor_score,paged_decode_attn_tiled,attention_finalize}.cu (one thread per output element /
// one CTA per (sequence, query head) there).
#include "common.cuh"

namespace {

constexpr int kMaxG = 8;          // query heads per kv head

__device__ __forceinline__ float e4m3_to_f(uint8_t b) {
  __nv_fp8_e4m3 v;
  v.__x = b;
  return float(v);
}

// EPL consecutive elements of a row, starting at element `at`, widened to fp32
template <int EPL, bool FP8>
__device__ __forceinline__ void load_row(const void* base, size_t at, float scale, float (&v)[EPL]) {
  if constexpr (FP8) {
    const uint8_t* p = static_cast<const uint8_t*>(base) + at;
    if constexpr (EPL == 4) {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = e4m3_to_f((w >> (8 * j)) & 0xff) * scale;
    } else {
      const uint2 w = *reinterpret_cast<const uint2*>(p);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[j] = e4m3_to_f((w.x >> (8 * j)) & 0xff) * scale;
        v[4 + j] = e4m3_to_f((w.y >> (8 * j)) & 0xff) * scale;
      }
    }
  } else {
    const __nv_bfloat16* p = static_cast<const __nv_bfloat16*>(base) + at;
    if constexpr (EPL == 4) {
      const uint2 w = *reinterpret_cast<const uint2*>(p);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
      }
    } else {
      const uint4 w = *reinterpret_cast<const uint4*>(p);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
      }
    }
  }
}

struct TileArgs {
  const __nv_bfloat16* q;      // [seqs, Hq, D]
  const void* k_pool;          // element strides below; bf16 or e4m3
  const void* v_pool;
  const int* tile_blocks;      // [seqs, cap] block ids into the pools
  const int* tile_counts;      // [seqs] blocks of this tile
  const int* last_valid;       // [seqs] token slots used in the tile's last block (null: all)
  float* m_state;              // [seqs, Hq]
  float* l_state;              // [seqs, Hq]
  float* o_state;              // [seqs, Hq, D]
  __nv_bfloat16* out;          // [seqs, Hq, D] or null
  int Hq, Hkv, block_size, cap;
  long long blk_stride, tok_stride, kvh_stride;
  float scale, k_scale, v_scale;
};

template <int D>
constexpr int tile_warps() { return D == 128 ? 8 : 4; }        // the merge buffer o_s must stay under 48 KB

template <int D, bool FP8>
__global__ void __launch_bounds__(tile_warps<D>() * 32) kv_tile_attn_kernel(const TileArgs a) {
  constexpr int EPL = D / 32;
  constexpr int kTileWarps = tile_warps<D>();
  const int kh = blockIdx.x, seq = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.Hq / a.Hkv;
  const int h0 = kh * G;

  __shared__ float m_s[kTileWarps][kMaxG], l_s[kTileWarps][kMaxG];
  __shared__ float o_s[kTileWarps][kMaxG][D];
  __shared__ float m_new[kMaxG], l_new[kMaxG];

  float q[kMaxG][EPL], o[kMaxG][EPL], m[kMaxG], l[kMaxG];
#pragma unroll
  for (int g = 0; g < kMaxG; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[g][e] = 0.f;
    if (g < G) {
      load_row<EPL, false>(a.q, ((size_t)seq * a.Hq + h0 + g) * D + lane * EPL, 1.f, q[g]);
#pragma unroll
      for (int e = 0; e < EPL; ++e) q[g][e] *= a.scale;
    } else {
#pragma unroll
      for (int e = 0; e < EPL; ++e) q[g][e] = 0.f;
    }
  }

  const int nblk = a.tile_counts[seq];
  int ntok = 0;
  if (nblk > 0) {
    int lv = a.last_valid ? a.last_valid[seq] : a.block_size;
    lv = lv < a.block_size ? (lv < 0 ? 0 : lv) : a.block_size;
    ntok = (nblk - 1) * a.block_size + lv;
  }
  // the next token's K / V rows are fetched before the current token is folded in, so the global-load latency
  // overlaps the dot products and shuffles of the previous token
  auto fetch = [&](int t, float (&kv)[EPL], float (&vv)[EPL]) {
    const int b = t / a.block_size, slot = t - b * a.block_size;
    const long long blk = a.tile_blocks[(size_t)seq * a.cap + b];
    const size_t at = (size_t)(blk * a.blk_stride + slot * a.tok_stride + kh * a.kvh_stride) + lane * EPL;
    load_row<EPL, FP8>(a.k_pool, at, a.k_scale, kv);
    load_row<EPL, FP8>(a.v_pool, at, a.v_scale, vv);
  };
  float kn[EPL], vn[EPL];
  if (warp < ntok) fetch(warp, kn, vn);
  for (int t = warp; t < ntok; t += kTileWarps) {
    float kv[EPL], vv[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      kv[e] = kn[e];
      vv[e] = vn[e];
    }
    if (t + kTileWarps < ntok) fetch(t + kTileWarps, kn, vn);
#pragma unroll
    for (int g = 0; g < kMaxG; ++g) {
      if (g < G) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) s = fmaf(q[g][e], kv[e], s);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        const float mn = fmaxf(m[g], s);
        const float c_old = __expf(m[g] - mn), c_new = __expf(s - mn);
        l[g] = l[g] * c_old + c_new;
#pragma unroll
        for (int e = 0; e < EPL; ++e) o[g][e] = o[g][e] * c_old + vv[e] * c_new;
        m[g] = mn;
      }
    }
  }
#pragma unroll
  for (int g = 0; g < kMaxG; ++g) {
    if (g < G) {
      if (lane == 0) {
        m_s[warp][g] = m[g];
        l_s[warp][g] = l[g];
      }
#pragma unroll
      for (int e = 0; e < EPL; ++e) o_s[warp][g][lane * EPL + e] = o[g][e];
    }
  }
  __syncthreads();
  // merge the warps' partial states with the running state of earlier tiles
  for (int i = threadIdx.x; i < G * D; i += kTileWarps * 32) {
    const int g = i / D, d = i - g * D;
    const size_t hs = (size_t)seq * a.Hq + h0 + g;
    const float m0 = a.m_state[hs];
    float M = m0;
#pragma unroll
    for (int w = 0; w < kTileWarps; ++w) M = fmaxf(M, m_s[w][g]);
    float L = 0.f, O = 0.f;
    if (M > -INFINITY) {
      const float c0 = m0 > -INFINITY ? __expf(m0 - M) : 0.f;
      L = a.l_state[hs] * c0;
      O = a.o_state[hs * D + d] * c0;
#pragma unroll
      for (int w = 0; w < kTileWarps; ++w) {
        const float c = m_s[w][g] > -INFINITY ? __expf(m_s[w][g] - M) : 0.f;
        L += l_s[w][g] * c;
        O += o_s[w][g][d] * c;
      }
    }
    a.o_state[hs * D + d] = O;
    if (a.out) a.out[hs * D + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
    // every thread of a head computes the same (M, L); the one at d == 0 keeps them for the store
    // after the barrier, once no thread reads the old running state any more
    if (d == 0) {
      m_new[g] = M;
      l_new[g] = L;
    }
  }
  __syncthreads();
  for (int g = threadIdx.x; g < G; g += kTileWarps * 32) {
    const size_t hs = (size_t)seq * a.Hq + h0 + g;
    a.m_state[hs] = m_new[g];
    a.l_state[hs] = l_new[g];
  }
}

__global__ void attn_finalize_kernel(const float* __restrict__ l_state, const float* __restrict__ o_state,
                                     __nv_bfloat16* __restrict__ out, long long n, int D) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float l = l_state[i / D];
  out[i] = __float2bfloat16(l > 0.f ? o_state[i] / l : 0.f);
}

struct ProjArgs {
  const void* x;               // flat rows [R, D] or a paged pool
  const __nv_bfloat16* P;      // [D, r]
  __nv_bfloat16* out;
  const int* src_blocks;       // null: flat rows; else pool block of each projected block
  const int* dst_blocks;       // destination block index of each projected block
  long long rows;
  int D, r, Hkv, block_size;
  long long blk_stride, tok_stride, kvh_stride;
  float scale;
};

constexpr int kProjWarps = 8;

template <bool FP8>
__global__ void __launch_bounds__(kProjWarps * 32) lowrank_project_kernel(const ProjArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Ps = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [D][r]
  float* xs = reinterpret_cast<float*>(smem_raw + (size_t)a.D * a.r * 2);         // [warps][D]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < a.D * a.r; i += blockDim.x) Ps[i] = a.P[i];
  __syncthreads();
  float* xw = xs + warp * a.D;
  for (long long row = (long long)blockIdx.x * kProjWarps + warp; row < a.rows;
       row += (long long)gridDim.x * kProjWarps) {
    size_t src, dst;
    if (a.src_blocks) {
      const int per = a.block_size * a.Hkv;
      const long long j = row / per;
      const int rem = (int)(row - j * per);
      const int tok = rem / a.Hkv, h = rem - tok * a.Hkv;
      src = (size_t)((long long)a.src_blocks[j] * a.blk_stride + tok * a.tok_stride + h * a.kvh_stride);
      dst = (((size_t)a.dst_blocks[j] * a.Hkv + h) * a.block_size + tok) * a.r;
    } else {
      src = (size_t)row * a.D;
      dst = (size_t)row * a.r;
    }
    for (int i = lane; i < a.D; i += 32) {
      float v;
      if constexpr (FP8) v = e4m3_to_f(static_cast<const uint8_t*>(a.x)[src + i]) * a.scale;
      else v = __bfloat162float(static_cast<const __nv_bfloat16*>(a.x)[src + i]);
      xw[i] = v;
    }
    __syncwarp();
    for (int j = lane; j < a.r; j += 32) {
      float acc = 0.f;
      for (int i = 0; i < a.D; ++i) acc = fmaf(xw[i], __bfloat162float(Ps[i * a.r + j]), acc);
      a.out[dst + j] = __float2bfloat16(acc);
    }
    __syncwarp();
  }
}

struct ScoreArgs {
  const __nv_bfloat16* q_lr;   // [seqs, Hq, r]
  const __nv_bfloat16* k_lr;   // [blocks, Hkv, block_size, r]
  const int* blocks;           // [seqs, cap] indices into k_lr
  const int* counts;           // [seqs]
  const int* last_valid;       // [seqs] or null
  float* scores;               // [seqs, cap]
  int Hq, Hkv, block_size, r, cap;
};

constexpr int kMaxR = 64;

__global__ void __launch_bounds__(128) predictor_score_kernel(const ScoreArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* qs = reinterpret_cast<float*>(smem_raw);                                   // [Hq][r]
  __shared__ float wmax[4];
  const int b = blockIdx.x, seq = blockIdx.y;
  const int n = a.counts[seq];
  if (b >= n) {
    if (threadIdx.x == 0) a.scores[(size_t)seq * a.cap + b] = -INFINITY;
    return;
  }
  for (int i = threadIdx.x; i < a.Hq * a.r; i += blockDim.x)
    qs[i] = __bfloat162float(a.q_lr[(size_t)seq * a.Hq * a.r + i]);
  __syncthreads();
  const int G = a.Hq / a.Hkv;
  int toks = a.block_size;
  if (b == n - 1 && a.last_valid) toks = min(max(a.last_valid[seq], 0), a.block_size);
  const __nv_bfloat16* kb = a.k_lr + (size_t)a.blocks[(size_t)seq * a.cap + b] * a.Hkv * a.block_size * a.r;
  float best = -INFINITY;
  for (int p = threadIdx.x; p < a.Hkv * a.block_size; p += blockDim.x) {
    const int h = p / a.block_size, tok = p - h * a.block_size;
    if (tok >= toks) continue;
    float k[kMaxR];
    const __nv_bfloat16* kr = kb + (size_t)p * a.r;
#pragma unroll
    for (int i = 0; i < kMaxR; ++i) k[i] = i < a.r ? __bfloat162float(kr[i]) : 0.f;
    for (int g = 0; g < G; ++g) {
      const float* qr = qs + (h * G + g) * a.r;
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxR; ++i)
        if (i < a.r) dot = fmaf(qr[i], k[i], dot);
      best = fmaxf(best, dot);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, off));
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0)
    a.scores[(size_t)seq * a.cap + b] = fmaxf(fmaxf(wmax[0], wmax[1]), fmaxf(wmax[2], wmax[3]));
}

}  // namespace

struct MbKvTileArgs {
  const void* q;
  const void* k_pool;
  const void* v_pool;
  const void* tile_blocks;
  const void* tile_counts;
  const void* last_valid;
  void* m_state;
  void* l_state;
  void* o_state;
  void* out;
  int num_seqs, Hq, Hkv, D, block_size, cap, kv_fp8;
  long long blk_stride, tok_stride, kvh_stride;
  float scale, k_scale, v_scale;
};

extern "C" int mb_kv_tile_attn(const MbKvTileArgs* p, cudaStream_t stream) {
  if (!p || p->num_seqs <= 0 || p->Hkv <= 0 || p->Hq % p->Hkv || p->Hq / p->Hkv > kMaxG) return MB_ERR_BAD_ARG;
  if (p->D != 128 && p->D != 256) return MB_ERR_UNSUPPORTED;
  // every row start must keep the lanes' 8- / 16-byte loads aligned
  const int unit = p->D / 32;      // elements per load
  if (p->blk_stride % unit || p->tok_stride % unit || p->kvh_stride % unit) return MB_ERR_BAD_ARG;
  TileArgs a{static_cast<const __nv_bfloat16*>(p->q), p->k_pool, p->v_pool,
             static_cast<const int*>(p->tile_blocks), static_cast<const int*>(p->tile_counts),
             static_cast<const int*>(p->last_valid), static_cast<float*>(p->m_state),
             static_cast<float*>(p->l_state), static_cast<float*>(p->o_state),
             static_cast<__nv_bfloat16*>(p->out), p->Hq, p->Hkv, p->block_size, p->cap,
             p->blk_stride, p->tok_stride, p->kvh_stride, p->scale, p->k_scale, p->v_scale};
  const dim3 grid(p->Hkv, p->num_seqs);
  if (p->D == 128) {
    if (p->kv_fp8) kv_tile_attn_kernel<128, true><<<grid, tile_warps<128>() * 32, 0, stream>>>(a);
    else kv_tile_attn_kernel<128, false><<<grid, tile_warps<128>() * 32, 0, stream>>>(a);
  } else {
    if (p->kv_fp8) kv_tile_attn_kernel<256, true><<<grid, tile_warps<256>() * 32, 0, stream>>>(a);
    else kv_tile_attn_kernel<256, false><<<grid, tile_warps<256>() * 32, 0, stream>>>(a);
  }
  return (int)cudaGetLastError();
}

extern "C" int mb_attn_finalize(const void* l_state, const void* o_state, void* out, long long heads, int D,
                                cudaStream_t stream) {
  if (heads <= 0 || D <= 0) return MB_ERR_BAD_ARG;
  const long long n = heads * D;
  attn_finalize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
      static_cast<const float*>(l_state), static_cast<const float*>(o_state), static_cast<__nv_bfloat16*>(out), n, D);
  return (int)cudaGetLastError();
}

struct MbLowrankArgs {
  const void* x;
  const void* P;
  void* out;
  const void* src_blocks;
  const void* dst_blocks;
  long long rows;
  int D, r, Hkv, block_size, fp8;
  long long blk_stride, tok_stride, kvh_stride;
  float scale;
};

extern "C" int mb_lowrank_project(const MbLowrankArgs* p, cudaStream_t stream) {
  if (!p || p->rows <= 0 || p->D <= 0 || p->D > 512 || p->r <= 0 || p->r > kMaxR) return MB_ERR_BAD_ARG;
  if (p->src_blocks && (p->Hkv <= 0 || p->block_size <= 0 || !p->dst_blocks)) return MB_ERR_BAD_ARG;
  ProjArgs a{p->x, static_cast<const __nv_bfloat16*>(p->P), static_cast<__nv_bfloat16*>(p->out),
             static_cast<const int*>(p->src_blocks), static_cast<const int*>(p->dst_blocks), p->rows, p->D, p->r,
             p->Hkv, p->block_size, p->blk_stride, p->tok_stride, p->kvh_stride, p->scale};
  const size_t smem = (size_t)p->D * p->r * 2 + (size_t)kProjWarps * p->D * 4;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(lowrank_project_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(lowrank_project_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  long long ctas = (p->rows + kProjWarps - 1) / kProjWarps;
  if (ctas > 148 * 8) ctas = 148 * 8;
  if (p->fp8) lowrank_project_kernel<true><<<(unsigned)ctas, kProjWarps * 32, smem, stream>>>(a);
  else lowrank_project_kernel<false><<<(unsigned)ctas, kProjWarps * 32, smem, stream>>>(a);
  return (int)cudaGetLastError();
}

struct MbScoreArgs {
  const void* q_lr;
  const void* k_lr;
  const void* blocks;
  const void* counts;
  const void* last_valid;
  void* scores;
  int num_seqs, Hq, Hkv, block_size, r, cap;
};

extern "C" int mb_predictor_score(const MbScoreArgs* p, cudaStream_t stream) {
  if (!p || p->num_seqs <= 0 || p->cap <= 0 || p->Hkv <= 0 || p->Hq % p->Hkv || p->r <= 0 || p->r > kMaxR)
    return MB_ERR_BAD_ARG;
  const size_t smem = (size_t)p->Hq * p->r * 4;
  if (smem > 48 * 1024) return MB_ERR_TOO_LARGE;
  ScoreArgs a{static_cast<const __nv_bfloat16*>(p->q_lr), static_cast<const __nv_bfloat16*>(p->k_lr),
              static_cast<const int*>(p->blocks), static_cast<const int*>(p->counts),
              static_cast<const int*>(p->last_valid), static_cast<float*>(p->scores), p->Hq, p->Hkv,
              p->block_size, p->r, p->cap};
  predictor_score_kernel<<<dim3(p->cap, p->num_seqs), 128, smem, stream>>>(a);
  return (int)cudaGetLastError();
}
