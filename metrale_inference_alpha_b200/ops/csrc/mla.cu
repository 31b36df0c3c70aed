// Absorbed multi-head latent attention (DeepSeek-V2/V3 shape) over the paged latent cache.
//
// Cache row per token: [kv_lora = 512 latent dims (RMS-normed) | 64 rope key dims], bf16, a single
// shared "kv head". Queries arrive already absorbed (q_nope * W_uk | rope(q_rope)), 576 dims per
// head. Scores use the whole 576-dim row, values are its first 512 dims, so this is multi-query
// attention in which K and V are the same bytes: a tile of cached rows is staged in shared memory
// once and feeds both products.
//
// grid (ceil(H * max_q_len / 16), num_seqs, parts), 128 threads. A CTA owns 16 query rows
// (row r of a sequence = query token r / H, head r % H) and one partition of the context.
// Per 64-token tile (cp.async, two stages):
//   S   warp w: S[16 rows x 16 tokens] for tokens 16w..16w+15, 36 k steps of mma.sync m16n8k16
//       (Q fragments by ldmatrix from shared memory: 576 dims do not fit registers);
//   softmax over the tile with the row maximum shared by the four warps (shared memory), P -> bf16
//       in shared memory;
//   O   warp w: O[16 rows x 128 latent dims 128w..] += P[16 x 64] * V[64 x 128] (ldmatrix.trans).
// Partitions are merged by mla_merge_kernel. Rows of 1152 bytes are XOR-swizzled in 16-byte
// chunks so that ldmatrix sees no bank conflicts.
//
// Reference behaviour: kernels/gb10/deepseek-v4-flash/nvfp4/{paged_decode_attn_mla.cu,
// mla_paged_decode_fp8.cu, mla_absorbed.cu} (CUDA-core per-head loops there).
#include "common.cuh"
#include "mla_args.h"

namespace {

constexpr int kD = 576, kL = 512, kRowB = kD * 2, kChunks = kRowB / 16, kTile = 64;
constexpr int kTileB = kTile * kRowB;
constexpr int kQB = 16 * kRowB;
constexpr int kSmem = 2 * kTileB + kQB + 16 * 128 /*P*/ + 4 * 16 * 4 /*max*/ + 4 * 16 * 4 /*l*/;

struct MlaParams {
  const __nv_bfloat16* q;       // [rows, H, 576]
  const __nv_bfloat16* cache;   // [num_blocks, block_size, 1, 576]
  const int* block_table;
  int max_blocks;
  const int* q_start;
  const int* q_len;
  const int* ctx_len;
  int H, block_size;
  long long num_blocks;
  float scale;
  float* out;                   // [rows, H, 512] fp32
  float* part_o;                // [rows * H, parts, 512]
  float* part_ml;               // [rows * H, parts, 2]
  int parts, part_tokens;
  uint32_t* status;
};

__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return (uint32_t)(row * kRowB + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ void ldsm4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(128, 1) mla_decode_kernel(const MlaParams p) {
  extern __shared__ __align__(128) uint8_t smem_mla[];
  const uint32_t sbase = mb::smem_u32(smem_mla);
  const uint32_t sQ = sbase + 2 * kTileB, sP = sQ + kQB;
  float* s_max = reinterpret_cast<float*>(smem_mla + 2 * kTileB + kQB + 16 * 128);
  float* s_l = s_max + 64;
  const int rg = blockIdx.x, seq = blockIdx.y, part = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int qlen = p.q_len[seq], ctx = p.ctx_len[seq], qs = p.q_start[seq];
  const int R = p.H * qlen;
  if (qlen <= 0 || rg * 16 >= R) return;
  const int nparts = max(1, (ctx + p.part_tokens - 1) / p.part_tokens);
  if (part >= nparts) return;
  const int part_len = (((ctx + nparts - 1) / nparts) + 63) & ~63;
  const int tok_begin = part * part_len;
  const int tok_end = min(ctx, tok_begin + part_len);
  const int ntiles = tok_begin < tok_end ? (tok_end - tok_begin + kTile - 1) / kTile : 0;
  const int* bt = p.block_table + (size_t)seq * p.max_blocks;

  auto issue_tile = [&](int it) {
    const uint32_t dst = sbase + (it & 1) * kTileB;
    const int tok0 = tok_begin + it * kTile;
    for (int idx = tid; idx < kTile * kChunks; idx += 128) {
      const int r = idx / kChunks, c = idx - r * kChunks;
      const int tok = tok0 + r;
      int sz = 0;
      size_t off = 0;
      if (tok < tok_end) {
        long long blk = bt[tok / p.block_size];
        if (blk < 0 || blk >= p.num_blocks) {
          if (p.status) atomicCAS(p.status, 0u, MB_ST_BOUNDS);
          blk = 0;
        }
        off = ((size_t)blk * p.block_size + tok % p.block_size) * kRowB + (size_t)c * 16;
        sz = 16;
      }
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + swz(r, c)),
                   "l"(reinterpret_cast<const uint8_t*>(p.cache) + off), "r"(sz) : "memory");
    }
  };
  if (ntiles > 0) issue_tile(0);
  asm volatile("cp.async.commit_group;" ::: "memory");

  // Q rows of this group -> shared memory (zero rows past R)
  for (int idx = tid; idx < 16 * kChunks; idx += 128) {
    const int r = idx / kChunks, c = idx - r * kChunks;
    const int row = rg * 16 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < R) {
      const int tq = row / p.H, hh = row - tq * p.H;
      v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.q) +
                                          ((size_t)(qs + tq) * p.H + hh) * kRowB + (size_t)c * 16);
    }
    *reinterpret_cast<uint4*>(smem_mla + 2 * kTileB + swz(r, c)) = v;
  }

  float o_acc[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[n][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  int lim[2];
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    const int row = rg * 16 + g + hr * 8;
    lim[hr] = row < R ? ctx - qlen + row / p.H + 1 : 0;      // rows past R see nothing
  }
  const float sc_log2 = p.scale * 1.44269504088896f;

  for (int it = 0; it < ntiles; ++it) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (it + 1 < ntiles) issue_tile(it + 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const uint32_t kT = sbase + (it & 1) * kTileB;
    const int tok0 = tok_begin + it * kTile + warp * 16;

    // ---- S = Q K^T for this warp's 16 tokens
    float s[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
#pragma unroll 4
    for (int ks = 0; ks < kD / 16; ++ks) {
      uint32_t a[4], b[4];
      ldsm4(a, sQ + swz((lane & 7) + (((lane >> 3) & 1) << 3), ks * 2 + (lane >> 4)));
      ldsm4(b, kT + swz(warp * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
      mma_bf16(s[0], a, b[0], b[1]);
      mma_bf16(s[1], a, b[2], b[3]);
    }
    // ---- tile softmax; the row maximum is shared by the four warps
    float mx[2];
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      const int limit = min(lim[hr], tok_end);
      float m = -INFINITY;
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int tok = tok0 + n * 8 + t * 2 + i;
          float v = s[n][hr * 2 + i] * sc_log2;
          if (tok >= limit) v = -INFINITY;
          s[n][hr * 2 + i] = v;
          m = fmaxf(m, v);
        }
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      mx[hr] = m;
      if (t == 0) s_max[warp * 16 + g + hr * 8] = m;
    }
    __syncthreads();
    float alpha[2];
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      const int r = g + hr * 8;
      const float tm = fmaxf(fmaxf(s_max[r], s_max[16 + r]), fmaxf(s_max[32 + r], s_max[48 + r]));
      const float m_new = fmaxf(m_run[hr], tm);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      alpha[hr] = ex2(m_run[hr] - m_use);
      float rs = 0.f;
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float pv = ex2(s[n][hr * 2 + i] - m_use);
          s[n][hr * 2 + i] = pv;
          rs += pv;
        }
      l_run[hr] = l_run[hr] * alpha[hr] + rs;       // this warp's tokens only; summed at the end
      m_run[hr] = m_new;
    }
    // P (bf16) -> shared memory [16 rows][64 tokens], 128-byte rows, swizzled
#pragma unroll
    for (int hr = 0; hr < 2; ++hr)
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const int r = g + hr * 8;
        const int col = warp * 16 + n * 8 + t * 2;                 // token column
        const uint32_t addr = sP + r * 128 + ((((col >> 3) ^ (r & 7)) << 4) | ((col & 7) << 1));
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(pack_bf16(s[n][hr * 2], s[n][hr * 2 + 1])) : "memory");
      }
    __syncthreads();
    // ---- O[:, 128 warp ..] = alpha * O + P V
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      o_acc[n][0] *= alpha[0]; o_acc[n][1] *= alpha[0];
      o_acc[n][2] *= alpha[1]; o_acc[n][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4];
      {
        const int r = (lane & 7) + (((lane >> 3) & 1) << 3);
        const int ch = kk * 2 + (lane >> 4);
        ldsm4(a, sP + r * 128 + ((ch ^ (r & 7)) << 4));
      }
#pragma unroll
      for (int n2 = 0; n2 < 8; ++n2) {
        uint32_t b[4];
        ldsm4t(b, kT + swz(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), warp * 16 + n2 * 2 + (lane >> 4)));
        mma_bf16(o_acc[n2 * 2], a, b[0], b[1]);
        mma_bf16(o_acc[n2 * 2 + 1], a, b[2], b[3]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // ---- row sums over the four warps, normalise, write
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    float l = l_run[hr];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (t == 0) s_l[warp * 16 + g + hr * 8] = l;
  }
  __syncthreads();
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    const int r = g + hr * 8;
    const int row = rg * 16 + r;
    if (row >= R) continue;
    const float l = s_l[r] + s_l[16 + r] + s_l[32 + r] + s_l[48 + r];
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const int tq = row / p.H, hh = row - tq * p.H;
    const size_t grow = (size_t)(qs + tq) * p.H + hh;
    float* dst = nparts == 1 ? p.out + grow * kL : p.part_o + (grow * p.parts + part) * kL;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      const float2 v = make_float2(o_acc[n][hr * 2] * inv, o_acc[n][hr * 2 + 1] * inv);
      *reinterpret_cast<float2*>(dst + warp * 128 + n * 8 + t * 2) = v;
    }
    if (nparts > 1 && warp == 0 && t == 0) {
      p.part_ml[(grow * p.parts + part) * 2] = m_run[hr];
      p.part_ml[(grow * p.parts + part) * 2 + 1] = l;
    }
  }
}

// one CTA per (query row, head): weights l_i * 2^(m_i - M), in partition order
__global__ void mla_merge_kernel(const MlaParams p, const int* row_seq) {
  const int grow = blockIdx.x;                      // (token row) * H + head
  const int seq = row_seq[grow / p.H];
  mb::pdl_wait();
  const int ctx = p.ctx_len[seq];
  const int nparts = max(1, (ctx + p.part_tokens - 1) / p.part_tokens);
  if (nparts == 1) return;                          // the decode kernel wrote the row directly
  float M = -INFINITY;
  for (int s = 0; s < nparts; ++s) M = fmaxf(M, p.part_ml[((size_t)grow * p.parts + s) * 2]);
  float wsum = 0.f;
  for (int s = 0; s < nparts; ++s) {
    const float m = p.part_ml[((size_t)grow * p.parts + s) * 2], l = p.part_ml[((size_t)grow * p.parts + s) * 2 + 1];
    wsum += m == -INFINITY ? 0.f : l * exp2f(m - M);
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  for (int d = threadIdx.x; d < kL; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < nparts; ++s) {
      const float m = p.part_ml[((size_t)grow * p.parts + s) * 2], l = p.part_ml[((size_t)grow * p.parts + s) * 2 + 1];
      const float w = m == -INFINITY ? 0.f : l * exp2f(m - M) * inv;
      acc += w * p.part_o[((size_t)grow * p.parts + s) * kL + d];
    }
    p.out[(size_t)grow * kL + d] = acc;
  }
}

// ------------------------------------------------------------------ decode on tcgen05 / TMEM
// One query token per sequence, all heads of it as the 128 rows of one UMMA tile: thread r owns head r.
// grid (2 halves of the 512 value dims, partitions of the context, sequences), 128 threads. Per tile of
// 32 cached tokens the latent rows [32 x 576] are staged ONCE (nine 64-dim blocks, 128-byte swizzle) and
// feed both products: S = Q K^T (M 128, N 32, 36 k steps over the 576 dims, K-major) and, for this CTA's
// half, O += P V (M 128, N 256, 2 k steps) with V = four of the same blocks read as an MN-major operand.
// S (32 columns) and O (256 columns) live in TMEM; O is rescaled only when a row maximum moves by more
// than 2^8; the next tile's rows are fetched into registers while the products run. Both halves compute
// the same S (the second one's tile reads hit L2). Partitions are merged by mla_merge_kernel.
constexpr int kTcT = 32;                       // cached tokens per tile
constexpr int kTcBlocks = kD / 64;             // 9 blocks of 64 dims
constexpr int kTcQB = 128 * 128;               // one Q block: 128 rows x 128 B
constexpr int kTcKB = kTcT * 128;              // one cache block of a tile: 32 rows x 128 B
constexpr int kTcSmem = kTcBlocks * (kTcQB + kTcKB) + 128 * 128 /*P*/ + 1024 /*alignment*/;

__device__ __forceinline__ uint32_t tc_sw(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }
__device__ __forceinline__ float tc_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(128, 1) mla_decode_tc_kernel(const MlaParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint8_t* sQ = smem_raw + ((1024u - (mb::smem_u32(smem_raw) & 1023u)) & 1023u);   // 9 x [128 rows x 128 B]
  uint8_t* sK = sQ + kTcBlocks * kTcQB;                                             // 9 x [32 tokens x 128 B]
  uint8_t* sP = sK + kTcBlocks * kTcKB;                                             // [128 rows x 128 B], 32 tokens used
  __shared__ uint64_t bar_s, bar_o;
  __shared__ uint32_t s_tmem;
  const int hv = blockIdx.x, part = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5;
  mb::pdl_wait();
  const int ctx = p.ctx_len[seq];
  if (p.q_len[seq] <= 0) return;
  const int nparts = max(1, (ctx + p.part_tokens - 1) / p.part_tokens);
  if (part >= nparts) return;
  const int tok_begin = part * p.part_tokens, tok_end = min(ctx, tok_begin + p.part_tokens);
  const int tiles = (tok_end - tok_begin + kTcT - 1) / kTcT;
  const int row = p.q_start[seq];                       // the sequence's single query row
  const int* bt = p.block_table + (size_t)seq * p.max_blocks;
  if (tid == 0) {
    mb::mbar_init(&bar_s, 1);
    mb::mbar_init(&bar_o, 1);
    mb::mbar_fence_init();
  }
  if (warp == 0) mb::tmem_alloc(&s_tmem, 512);
  {
    const uint4* src = tid < p.H ? reinterpret_cast<const uint4*>(p.q + ((size_t)row * p.H + tid) * kD) : nullptr;
#pragma unroll 8
    for (int c = 0; c < kChunks; ++c) {
      const uint4 v = src ? src[c] : make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(sQ + (c >> 3) * kTcQB + tc_sw(tid, c & 7)) = v;
    }
    // the upper half of every P row is never written again: the second product only reads 32 tokens
#pragma unroll
    for (int c = 4; c < 8; ++c) *reinterpret_cast<uint4*>(sP + tc_sw(tid, c)) = make_uint4(0, 0, 0, 0);
  }
  mb::tc_fence_before();
  __syncthreads();
  mb::tc_fence_after();
  mb::pdl_launch_dependents();                          // only once this CTA holds its TMEM columns
  const uint32_t tmem = s_tmem;
  const uint32_t t_row = tmem + ((uint32_t)(warp * 32) << 16);
  constexpr uint32_t kIdescS = mb::umma_idesc(1, 1, 128, kTcT);
  constexpr uint32_t kIdescO = mb::umma_idesc(1, 1, 128, 256, 0, 1);
  const uint32_t aQ = mb::smem_u32(sQ), aK = mb::smem_u32(sK), aP = mb::smem_u32(sP);
  const float sc_log2 = p.scale * 1.44269504088896f;
  float m_run = -INFINITY, l_run = 0.f;
  uint32_t ph_s = 0, ph_o = 0;
  bool ok = true;
  // staging: thread = (token tid / 4 of the tile, quarter tid % 4 of its row): 18 consecutive 16-byte chunks,
  // one block-table lookup per tile
  constexpr int kPer = kChunks / 4;
  const int s_tok = tid >> 2, s_c0 = (tid & 3) * kPer;
  uint4 raw[kPer];
  auto fetch = [&](int jt) {
    const int tok = tok_begin + jt * kTcT + s_tok;
    if (jt < tiles && tok < tok_end) {
      long long blk = bt[tok / p.block_size];
      if (blk < 0 || blk >= p.num_blocks) {
        if (p.status) atomicCAS(p.status, 0u, MB_ST_BOUNDS);
        blk = 0;
      }
      const uint4* src = reinterpret_cast<const uint4*>(p.cache + ((size_t)blk * p.block_size + (tok % p.block_size)) * kD) + s_c0;
#pragma unroll
      for (int i = 0; i < kPer; ++i) raw[i] = __ldg(src + i);
    } else {
#pragma unroll
      for (int i = 0; i < kPer; ++i) raw[i] = make_uint4(0, 0, 0, 0);
    }
  };
  fetch(0);
  for (int j = 0; j < tiles; ++j) {
    if (j > 0) {                                        // the previous tile's second product read sK and sP
      ok = mb::mbar_wait(&bar_o, ph_o, p.status, MB_ST_TIMEOUT_MMA) && ok;
      ph_o ^= 1;
      mb::tc_fence_after();
    }
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int c = s_c0 + i;
      *reinterpret_cast<uint4*>(sK + (c >> 3) * kTcKB + tc_sw(s_tok, c & 7)) = raw[i];
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mb::tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      mb::tc_fence_after();
#pragma unroll
      for (int b = 0; b < kTcBlocks; ++b)
#pragma unroll
        for (int s = 0; s < 4; ++s)
          mb::umma_f16(tmem, mb::umma_desc_sw128(aQ + b * kTcQB + s * 32), mb::umma_desc_sw128(aK + b * kTcKB + s * 32),
                       kIdescS, (b | s) != 0);
      mb::tc_commit(&bar_s);
    }
    fetch(j + 1);
    ok = mb::mbar_wait(&bar_s, ph_s, p.status, MB_ST_TIMEOUT_MMA) && ok;
    ph_s ^= 1;
    mb::tc_fence_after();
    {
      float sv[kTcT];
      mb::tmem_ld16(t_row, sv);
      mb::tmem_ld16(t_row + 16, sv + 16);
      float mx = -INFINITY;
      const int tok0 = tok_begin + j * kTcT;
#pragma unroll
      for (int i = 0; i < kTcT; ++i) {
        const float v = (tok0 + i < tok_end) ? sv[i] * sc_log2 : -INFINITY;
        sv[i] = v;
        mx = fmaxf(mx, v);
      }
      float alpha = 1.f;
      const bool move = mx > m_run + 8.f;
      if (move) {
        alpha = tc_ex2(m_run - mx);
        m_run = mx;
      }
      if (j > 0 && __any_sync(0xffffffffu, move)) {
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          float ov[16];
          mb::tmem_ld16(t_row + 32 + c * 16, ov);
#pragma unroll
          for (int i = 0; i < 16; ++i) ov[i] *= alpha;
          mb::tmem_st16(t_row + 32 + c * 16, ov);
        }
        mb::tmem_st_wait();
      }
      const float m_use = m_run == -INFINITY ? 0.f : m_run;
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 pk;
        uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = tc_ex2(sv[c * 8 + 2 * i] - m_use), b = tc_ex2(sv[c * 8 + 2 * i + 1] - m_use);
          const __nv_bfloat162 pb = __floats2bfloat162_rn(a, b);
          rs += a + b;
          pw[i] = *reinterpret_cast<const uint32_t*>(&pb);
        }
        *reinterpret_cast<uint4*>(sP + tc_sw(tid, c)) = pk;
      }
      l_run = l_run * alpha + rs;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mb::tc_fence_before();
    ok = __syncthreads_and(ok) != 0;
    if (!ok) break;
    if (tid == 0) {
      mb::tc_fence_after();
#pragma unroll
      for (int s = 0; s < 2; ++s)                         // 16 tokens per step = two 8-row groups of the tile
        mb::umma_f16(tmem + 32, mb::umma_desc_sw128(aP + s * 32),
                     mb::umma_desc_sw128_mn(aK + (4 * hv) * kTcKB + s * 2048, kTcKB, 1024), kIdescO, (j | s) != 0);
      mb::tc_commit(&bar_o);
    }
  }
  if (ok && tiles > 0) {
    ok = mb::mbar_wait(&bar_o, ph_o, p.status, MB_ST_TIMEOUT_MMA) && ok;
    mb::tc_fence_after();
  }
  if (ok) {                                               // uniform: tcgen05.ld is a whole-warp instruction
    const bool row_ok = tid < p.H;
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    const size_t grow = (size_t)row * p.H + (row_ok ? tid : 0);
    float* dst = (nparts == 1 ? p.out + grow * kL : p.part_o + (grow * p.parts + part) * kL) + hv * 256;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      float ov[16];
      mb::tmem_ld16(t_row + 32 + c * 16, ov);
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<float4*>(dst + c * 16 + i * 4) =
              make_float4(ov[4 * i] * inv, ov[4 * i + 1] * inv, ov[4 * i + 2] * inv, ov[4 * i + 3] * inv);
      }
    }
    if (row_ok && nparts > 1 && hv == 0) {
      p.part_ml[(grow * p.parts + part) * 2] = m_run;
      p.part_ml[(grow * p.parts + part) * 2 + 1] = l_run;
    }
  }
  mb::tc_fence_before();
  __syncthreads();
  if (warp == 0) mb::tmem_dealloc(tmem, 512);
}

}  // namespace

extern "C" {

// (MbMlaArgs: mla_args.h)

size_t mb_mla_ws_bytes(int total_rows, int H, int max_ctx, int part_tokens) {
  const int pt = part_tokens > 0 ? part_tokens : 1024;
  const size_t parts = (size_t)(max_ctx + pt - 1) / pt;
  return parts <= 1 ? 0 : (size_t)total_rows * H * parts * (kL + 2) * sizeof(float);
}

// Decode rows (one query token per sequence, H <= 128 heads) on the tcgen05 kernel; same arguments,
// workspace and results as mb_mla_attention.
int mb_mla_decode_tc(const MbMlaArgs* a, cudaStream_t stream) {
  if (!a || !a->q || !a->cache || !a->out || a->num_seqs <= 0 || a->H <= 0 || a->H > 128 || a->max_q_len != 1)
    return MB_ERR_BAD_ARG;
  MlaParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(a->q);
  p.cache = reinterpret_cast<const __nv_bfloat16*>(a->cache);
  p.block_table = a->block_table; p.max_blocks = a->max_blocks;
  p.q_start = a->q_start; p.q_len = a->q_len; p.ctx_len = a->ctx_len;
  p.H = a->H; p.block_size = a->block_size; p.num_blocks = a->num_blocks;
  p.scale = a->scale; p.out = a->out; p.status = a->status;
  p.part_tokens = a->part_tokens > 0 ? a->part_tokens : 1024;
  p.parts = (a->max_ctx + p.part_tokens - 1) / p.part_tokens;
  if (p.parts < 1) p.parts = 1;
  if (p.parts > 1) {
    const size_t need = mb_mla_ws_bytes(a->total_rows, a->H, a->max_ctx, p.part_tokens);
    if (!a->ws || a->ws_bytes < need || !a->row_seq) return MB_ERR_TOO_LARGE;
    p.part_o = reinterpret_cast<float*>(a->ws);
    p.part_ml = p.part_o + (size_t)a->total_rows * a->H * p.parts * kL;
  }
  if (p.parts > 65535) return MB_ERR_TOO_LARGE;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(mla_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaError_t e = mb::launch_kernel(mla_decode_tc_kernel, dim3(2, p.parts, a->num_seqs), dim3(128), (size_t)kTcSmem, stream, p);
  if (e != cudaSuccess) return (int)e;
  if (p.parts > 1) {
    e = mb::launch_kernel(mla_merge_kernel, dim3(a->total_rows * a->H), dim3(128), (size_t)0, stream, p, a->row_seq);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

int mb_mla_attention(const MbMlaArgs* a, cudaStream_t stream) {
  if (!a || !a->q || !a->cache || !a->out || a->num_seqs <= 0 || a->H <= 0 || a->max_q_len <= 0) return MB_ERR_BAD_ARG;
  if (a->impl == 2 || (a->impl == 0 && a->max_q_len == 1 && a->H <= 128 && a->H >= 16)) return mb_mla_decode_tc(a, stream);
  MlaParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(a->q);
  p.cache = reinterpret_cast<const __nv_bfloat16*>(a->cache);
  p.block_table = a->block_table; p.max_blocks = a->max_blocks;
  p.q_start = a->q_start; p.q_len = a->q_len; p.ctx_len = a->ctx_len;
  p.H = a->H; p.block_size = a->block_size; p.num_blocks = a->num_blocks;
  p.scale = a->scale; p.out = a->out; p.status = a->status;
  p.part_tokens = a->part_tokens > 0 ? a->part_tokens : 1024;
  p.parts = (a->max_ctx + p.part_tokens - 1) / p.part_tokens;
  if (p.parts < 1) p.parts = 1;
  if (p.parts > 1) {
    const size_t need = mb_mla_ws_bytes(a->total_rows, a->H, a->max_ctx, p.part_tokens);
    if (!a->ws || a->ws_bytes < need || !a->row_seq) return MB_ERR_TOO_LARGE;
    p.part_o = reinterpret_cast<float*>(a->ws);
    p.part_ml = p.part_o + (size_t)a->total_rows * a->H * p.parts * kL;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int groups = (a->H * a->max_q_len + 15) / 16;
  cudaError_t e = mb::launch_kernel(mla_decode_kernel, dim3(groups, a->num_seqs, p.parts), dim3(128), (size_t)kSmem, stream, p);
  if (e != cudaSuccess) return (int)e;
  if (p.parts > 1) {
    e = mb::launch_kernel(mla_merge_kernel, dim3(a->total_rows * a->H), dim3(128), (size_t)0, stream, p, a->row_seq);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

}  // extern "C"

// ------------------------------------------------------------------ absorbed-MLA operand assembly
// One launch between the projections and the attention kernel, replacing a chain of elementwise
// tensor ops: per token
//   * the compressed KV row [latent (L) | rope key (R)] from the kv_a projection: RMSNorm of the
//     latent with its weight, NeoX rotation of the rope key at the token's position, both written
//     as one bf16 cache row at the token's slot (rows without a slot write nothing);
//   * the absorbed query row of every head, [q_lat (L) | rotated q_rope (R)]: q_lat comes from the
//     batched absorption product q_nope W_uk (laid out [H, T, L]), q_rope from the q projection.
// grid = T tokens, 256 threads. Reference behaviour: mla_cache_assemble and the rope half of
// mla_batched_gemv (kernels/gb10/deepseek-v4-flash/nvfp4/mla_absorbed.cu).
namespace {
struct MlaPrepParams {
  const __nv_bfloat16* q;        // [T, H, nope + R]
  const __nv_bfloat16* q_lat;    // [H, T, L]
  const __nv_bfloat16* ckv;      // [T, L + R]
  const __nv_bfloat16* norm_w;   // [L]
  const float* cos_tab;          // [max_pos, R / 2]
  const float* sin_tab;
  const int* positions;
  const long long* slots;
  __nv_bfloat16* cache;          // [num_slots, L + R]
  __nv_bfloat16* qq;             // [T, H, L + R]
  int T, H, nope, R, L, max_pos;
  long long num_slots;
  float eps;
  uint32_t* status;
};

__global__ void __launch_bounds__(256) mla_prepare_kernel(const MlaPrepParams p) {
  __shared__ float s_red[8];
  __shared__ float s_cs[2][64];                      // cos | sin of this position (R / 2 <= 64)
  const int t = blockIdx.x, tid = threadIdx.x;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int pos = min(max(p.positions[t], 0), p.max_pos - 1);
  const int half = p.R / 2;
  if (tid < half) {
    s_cs[0][tid] = p.cos_tab[(size_t)pos * half + tid];
    s_cs[1][tid] = p.sin_tab[(size_t)pos * half + tid];
  }
  // latent RMSNorm (fp32 statistics over L)
  const __nv_bfloat16* row = p.ckv + (size_t)t * (p.L + p.R);
  float ss = 0.f;
  for (int i = tid; i < p.L; i += 256) {
    const float v = __bfloat162float(row[i]);
    ss += v * v;
  }
  ss = mb::warp_sum(ss);
  if ((tid & 31) == 0) s_red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += s_red[w];
  const float rinv = rsqrtf(tot / (float)p.L + p.eps);
  const long long slot = p.slots[t];
  if (slot >= p.num_slots) {
    if (p.status && tid == 0) atomicCAS(p.status, 0u, MB_ST_BOUNDS);
  } else if (slot >= 0) {
    __nv_bfloat16* dst = p.cache + (size_t)slot * (p.L + p.R);
    for (int i = tid; i < p.L; i += 256)
      dst[i] = __float2bfloat16(__bfloat162float(row[i]) * rinv * __bfloat162float(p.norm_w[i]));
    if (tid < half) {
      const float x1 = __bfloat162float(row[p.L + tid]), x2 = __bfloat162float(row[p.L + half + tid]);
      dst[p.L + tid] = __float2bfloat16(x1 * s_cs[0][tid] - x2 * s_cs[1][tid]);
      dst[p.L + half + tid] = __float2bfloat16(x2 * s_cs[0][tid] + x1 * s_cs[1][tid]);
    }
  }
  // absorbed query rows: 16-byte copies of q_lat, then the rotated rope part
  const int W = p.L + p.R;
  const int chunks = p.L / 8;
  for (int i = tid; i < p.H * chunks; i += 256) {
    const int h = i / chunks, c = i - h * chunks;
    *reinterpret_cast<uint4*>(p.qq + ((size_t)t * p.H + h) * W + c * 8) =
        *reinterpret_cast<const uint4*>(p.q_lat + ((size_t)h * p.T + t) * p.L + c * 8);
  }
  for (int i = tid; i < p.H * half; i += 256) {
    const int h = i / half, j = i - h * half;
    const __nv_bfloat16* qr = p.q + ((size_t)t * p.H + h) * (p.nope + p.R) + p.nope;
    const float x1 = __bfloat162float(qr[j]), x2 = __bfloat162float(qr[half + j]);
    __nv_bfloat16* dst = p.qq + ((size_t)t * p.H + h) * W + p.L;
    dst[j] = __float2bfloat16(x1 * s_cs[0][j] - x2 * s_cs[1][j]);
    dst[half + j] = __float2bfloat16(x2 * s_cs[0][j] + x1 * s_cs[1][j]);
  }
}
}  // namespace

extern "C" int mb_mla_prepare(const void* q, const void* q_lat, const void* ckv, const void* norm_w,
                              const float* cos_tab, const float* sin_tab, const int* positions, const long long* slots,
                              void* cache, void* qq, int T, int H, int nope, int R, int L, int max_pos,
                              long long num_slots, float eps, uint32_t* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (R > 128 || (R & 1) || L % 8 != 0 || H <= 0) return MB_ERR_BAD_ARG;
  MlaPrepParams p;
  p.q = (const __nv_bfloat16*)q; p.q_lat = (const __nv_bfloat16*)q_lat; p.ckv = (const __nv_bfloat16*)ckv;
  p.norm_w = (const __nv_bfloat16*)norm_w; p.cos_tab = cos_tab; p.sin_tab = sin_tab;
  p.positions = positions; p.slots = slots; p.cache = (__nv_bfloat16*)cache; p.qq = (__nv_bfloat16*)qq;
  p.T = T; p.H = H; p.nope = nope; p.R = R; p.L = L; p.max_pos = max_pos; p.num_slots = num_slots;
  p.eps = eps; p.status = status;
  return (int)mb::launch_kernel(mla_prepare_kernel, dim3(T), dim3(256), (size_t)0, stream, p);
}
