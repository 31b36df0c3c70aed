// Paged attention for GQA models on sm_100a.
//
//   mb_qk_norm_rope_kvwrite  per-head RMSNorm (optional) + NeoX RoPE (optional, partial
//                            rotary) on q and k, then K/V rows scattered into the paged
//                            cache by slot id, bf16 or e4m3 with a per-tensor scale.
//   mb_paged_attention       one kernel family for decode (1 query token), speculative
//                            verify (a few query tokens) and chunked prefill (many):
//                              * "split-KV" kernel: a CTA owns one (kv head, sequence,
//                                512-token partition); its 4 warps each take 16 of every
//                                64 cached tokens, all G*q_len query rows ride in the
//                                m16 rows of the tensor-core tiles, warps merge through
//                                shared memory, partitions merge in a second kernel.
//                                The partition size is fixed, so the result for one
//                                sequence never depends on what else is in the batch.
//                              * "split-Q" kernel (prefill): a CTA owns 64 query rows of
//                                one (q head, sequence), 16 per warp, and walks the
//                                causal range of cached tokens FlashAttention-2 style.
// Cache layout (both K and V): [num_blocks, block_size, kv_heads, head_dim].
// e4m3 cache rows are widened to f16 while being staged into shared memory with an
// integer bit trick (exact, 2^-8 scale folded into the softmax/output scales); bf16
// caches are staged as they are. The contraction is mma.sync m16n8k16 (these kernels
// are bandwidth-bound on the KV stream; the query side has at most 64 rows).
//
// Reference behaviour covered: kernels/gb10/common/fused_k_norm_rope_cache.cu,
// reshape_and_cache.cu, rope.cu, paged_decode_attn{,_fp8,_bf16_gqa,_fp8_gqa}.cu
// (+ split-K reduce), prefill_paged_compute.cuh and attn_prefill_paged{,_fp8,_batched}.cu.
#include "common.cuh"

namespace {

// ------------------------------------------------------------------ rope + kv write
struct RopeKvParams {
  int M, Hq, Hkv, D, rot;
  const __nv_bfloat16* qkv;      // [M, qkv_ld]: q heads, then k heads, then v heads
  long long qkv_ld;
  int q_head_stride;             // D, or 2*D when an output gate is interleaved per head
  int k_off, v_off;              // element offsets of k / v inside a row
  const int* positions;          // [M]
  const long long* slots;        // [M] flat slot = block * block_size + offset; <0 skips
  const __nv_bfloat16* q_norm_w; // [D] or null
  const __nv_bfloat16* k_norm_w;
  int norm_plus_one;
  float eps;
  const float* cos_tab;          // [max_pos, rot/2] or null (no rope)
  const float* sin_tab;
  int max_pos;
  __nv_bfloat16* q_out;          // [M, Hq, D]
  void* k_cache;
  void* v_cache;
  int cache_fp8;
  const float* k_scale;          // per-tensor dequant multipliers (fp8 cache)
  const float* v_scale;
  long long num_slots;
  uint32_t* status;
  float* amax;                   // optional [2]: running max |k|, max |v| of the rows written (online scale calibration)
};

// In-place change of an e4m3 cache's per-tensor scale for the listed slots: value * old / new.
// Used once, when online calibration freezes its scale and rewrites what the window wrote.
__global__ void kv_rescale_kernel(uint8_t* cache, const long long* __restrict__ slots, int n, int row_elems,
                                  long long num_slots, float old_scale, const float* __restrict__ new_scale) {
  const int i = blockIdx.x;
  if (i >= n) return;
  const long long slot = slots[i];
  if (slot < 0 || slot >= num_slots) return;
  const float f = old_scale / *new_scale;
  uint8_t* row = cache + (size_t)slot * row_elems;
  for (int j = threadIdx.x; j < row_elems; j += blockDim.x) row[j] = mb::float_to_e4m3(mb::e4m3_to_float(row[j]) * f);
}

__global__ void __launch_bounds__(128) rope_kv_kernel(const RopeKvParams p) {
  const int m = blockIdx.x;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int head = blockIdx.y * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int Htot = p.Hq + 2 * p.Hkv;
  if (head >= Htot) return;
  const int D = p.D;
  const int per = D / 32;  // <= 8
  const __nv_bfloat16* src;
  int kind;  // 0 q, 1 k, 2 v
  int h;
  if (head < p.Hq) { kind = 0; h = head; src = p.qkv + (size_t)m * p.qkv_ld + (size_t)h * p.q_head_stride; }
  else if (head < p.Hq + p.Hkv) { kind = 1; h = head - p.Hq; src = p.qkv + (size_t)m * p.qkv_ld + p.k_off + (size_t)h * D; }
  else { kind = 2; h = head - p.Hq - p.Hkv; src = p.qkv + (size_t)m * p.qkv_ld + p.v_off + (size_t)h * D; }

  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = j < per ? __bfloat162float(src[lane + 32 * j]) : 0.f;

  if (kind != 2) {
    const __nv_bfloat16* nw = kind == 0 ? p.q_norm_w : p.k_norm_w;
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
      ss = mb::warp_sum(ss);
      const float inv = rsqrtf(ss / (float)D + p.eps);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < per) {
          float w = __bfloat162float(nw[lane + 32 * j]);
          if (p.norm_plus_one) w += 1.f;
          // the normalised value passes through bf16 like an unfused norm kernel's output
          v[j] = __bfloat162float(__float2bfloat16(v[j] * inv * w));
        }
    }
    if (p.cos_tab) {
      int pos = p.positions[m];
      if (pos < 0 || pos >= p.max_pos) {
        if (lane == 0 && p.status) atomicCAS(p.status, 0u, MB_ST_BOUNDS);
        pos = 0;
      }
      const int half = p.rot / 2;       // a multiple of 32, or 16 (32 rotated dims)
      const int hj = half / 32;         // register distance between pair members
      const float* c = p.cos_tab + (size_t)pos * half;
      const float* s = p.sin_tab + (size_t)pos * half;
      if (half == 16) {
        // both members of a pair sit in register 0, sixteen lanes apart
        const float other = __shfl_xor_sync(0xffffffffu, v[0], 16);
        const int i = lane & 15;
        const float cs = c[i], sn = s[i];
        v[0] = lane < 16 ? v[0] * cs - other * sn : v[0] * cs + other * sn;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (j < hj) {
          const int i = lane + 32 * j;
          const float x1 = v[j], x2 = v[j + hj];
          const float cs = c[i], sn = s[i];
          v[j] = x1 * cs - x2 * sn;
          v[j + hj] = x2 * cs + x1 * sn;
        }
    }
  }

  if (kind == 0) {
    __nv_bfloat16* dst = p.q_out + ((size_t)m * p.Hq + h) * D;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < per) dst[lane + 32 * j] = __float2bfloat16(v[j]);
    return;
  }
  const long long slot = p.slots[m];
  if (slot < 0) return;
  if (slot >= p.num_slots) {
    if (lane == 0 && p.status) atomicCAS(p.status, 0u, MB_ST_BOUNDS);
    return;
  }
  const size_t off = ((size_t)slot * p.Hkv + h) * D;
  if (p.amax) {
    float mx = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(v[j]));
    mx = mb::warp_max(mx);
    // non-negative floats order like their bit patterns
    if (lane == 0) atomicMax(reinterpret_cast<int*>(p.amax + (kind - 1)), __float_as_int(mx));
  }
  if (p.cache_fp8) {
    const float sc = kind == 1 ? *p.k_scale : *p.v_scale;
    const float inv = 1.f / sc;
    uint8_t* dst = reinterpret_cast<uint8_t*>(kind == 1 ? p.k_cache : p.v_cache) + off;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < per) dst[lane + 32 * j] = mb::float_to_e4m3(v[j] * inv);
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(kind == 1 ? p.k_cache : p.v_cache) + off;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < per) dst[lane + 32 * j] = __float2bfloat16(v[j]);
  }
}

// ------------------------------------------------------------------ mma helpers
template <bool F16>
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  if constexpr (F16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}
__device__ __forceinline__ void ldsm4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
template <bool F16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (F16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}
// two e4m3 bytes (low 16 bits of x) -> f16x2 holding value * 2^-8 (exact, incl. denormals)
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2_scaled(uint32_t x) {
  const uint32_t w = __byte_perm(x, 0, 0x1404);  // b0 -> bits 15:8, b1 -> bits 31:24
  return (w & 0x80008000u) | ((w & 0x7F007F00u) >> 1);
}
// Shared-memory tile of 16-bit elements, rows of D elements, 16-byte chunks XOR-swizzled by
// (row & 7) so ldmatrix row fetches spread over all banks.
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

constexpr size_t kAttnCntBytes = 64 * 1024;   // arrival counters at the head of the split-KV workspace

struct AttnParams {
  const __nv_bfloat16* q;   // [rows, Hq, D]
  const void* k_cache;
  const void* v_cache;
  const int* block_table;   // [num_seqs, max_blocks]
  int max_blocks;
  const int* q_start;       // [num_seqs] first query row of the sequence
  const int* q_len;         // [num_seqs]
  const int* ctx_len;       // [num_seqs] cached tokens including this step's
  int Hq, Hkv, block_size;
  long long num_blocks;
  float scale;              // softmax scale
  const float* k_scale;
  const float* v_scale;
  __nv_bfloat16* out;       // [rows, Hq, D]
  float* part_o;            // [rows, Hq, parts, D]
  float* part_ml;           // [rows, Hq, parts, 2]
  int parts, part_tokens;
  uint32_t* part_cnt;       // [num_seqs * Hkv] arrival counters (zero between launches)
  int window;               // sliding window (0 = none)
  uint32_t* status;
  // optional NVFP4 output for the o projection (split-KV kernel, head_dim % 128 == 0): packed e2m1
  // [rows, ldq] + tiled ue4m3 scale factors, quantised with a calibrated global scale
  uint8_t* outq;
  int ldq;
  uint8_t* outq_sf;
  int outq_sf_k64;
  float outq_gs;
};

// Final store of four consecutive dims (c4 * 4 ..) of output row `orow` = token * Hq + head. In the
// quantised mode the four lanes that share a 16-dim block agree on its scale with two shuffles;
// every lane of the warp must call this (the callers' loops run whole warps when D % 128 == 0).
template <int D>
__device__ __forceinline__ void store_out4(const AttnParams& p, size_t orow, int c4, float a, float b, float c, float d) {
  if (p.outq) {
    float bmax = fmaxf(fmaxf(fabsf(a), fabsf(b)), fmaxf(fabsf(c), fabsf(d)));
    bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));
    bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 2));
    const uint8_t sfc = mb::float_to_e4m3(bmax / (6.f * p.outq_gs));
    const float sff = mb::e4m3_to_float(sfc);
    const float qi = sff > 0.f ? __fdividef(1.f, sff * p.outq_gs) : 0.f;
    const uint32_t w = mb::e2m1x2_pack(a * qi, b * qi) | (mb::e2m1x2_pack(c * qi, d * qi) << 8);
    const size_t m = orow / p.Hq;
    const int col = (int)(orow - m * p.Hq) * D + c4 * 4;             // index along the consumer's K
    *reinterpret_cast<uint16_t*>(p.outq + m * p.ldq + (col >> 1)) = (uint16_t)w;
    if ((c4 & 3) == 0) {
      const int kb = col >> 4;
      p.outq_sf[((m >> 7) * p.outq_sf_k64 + (kb >> 2)) * 512 + mb::sf_tile_offset((uint32_t)(m & 127), kb & 3)] = sfc;
    }
    return;
  }
  __nv_bfloat16* dst = p.out + orow * D + c4 * 4;
  *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(a, b);
  *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(c, d);
}

// Stage a [64 x D] tile of cache rows for one kv head into shared memory.
//   e4m3 cache: fetch() issues the global loads into registers, commit() widens to f16
//               and stores into the tile (register prefetch across the compute phase);
//   bf16 cache: fetch() issues cp.async straight into the tile, commit() waits for them.
template <int D, bool FP8>
struct TileLoader {
  static constexpr int kChunkElems = FP8 ? 16 : 8;           // elements per 16-byte load
  static constexpr int kChunksPerRow = D / kChunkElems;
  static constexpr int kTotal = 64 * kChunksPerRow;
  static constexpr int kPerThread = kTotal / 128;
  uint4 regs[FP8 ? kPerThread : 1];
  __device__ __forceinline__ void fetch(const AttnParams& p, const void* cache, const int* bt,
                                        int kv_head, int tok0, int tok_end, int tid,
                                        uint32_t smem_tile) {
    const int esize = FP8 ? 1 : 2;
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int idx = tid + i * 128;
      const int r = idx / kChunksPerRow, c = idx - r * kChunksPerRow;
      const int tok = tok0 + r;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(cache);
      bool valid = tok < tok_end;
      if (valid) {
        long long blk = bt[tok / p.block_size];
        if (blk < 0 || blk >= p.num_blocks) {
          if (p.status) atomicCAS(p.status, 0u, MB_ST_BOUNDS);
          valid = false;
        } else {
          src += (((size_t)blk * p.block_size + (tok % p.block_size)) * p.Hkv + kv_head) * D * esize +
                 (size_t)c * 16;
        }
      }
      if constexpr (FP8) {
        regs[i] = valid ? __ldg(reinterpret_cast<const uint4*>(src)) : make_uint4(0, 0, 0, 0);
      } else {
        const uint32_t dst = smem_tile + tile_off<D>(r, c);
        const int sz = valid ? 16 : 0;                        // 0 -> zero fill
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz)
                     : "memory");
      }
    }
    if constexpr (!FP8) asm volatile("cp.async.commit_group;" ::: "memory");
  }
  __device__ __forceinline__ void commit(uint32_t smem_tile, int tid) {
    if constexpr (!FP8) {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      return;
    } else {
#pragma unroll
      for (int i = 0; i < kPerThread; ++i) {
        const int idx = tid + i * 128;
        const int r = idx / kChunksPerRow, c = idx - r * kChunksPerRow;
        const uint4 v = regs[i];
        uint4 lo, hi;
        lo.x = e4m3x2_to_f16x2_scaled(v.x);
        lo.y = e4m3x2_to_f16x2_scaled(v.x >> 16);
        lo.z = e4m3x2_to_f16x2_scaled(v.y);
        lo.w = e4m3x2_to_f16x2_scaled(v.y >> 16);
        hi.x = e4m3x2_to_f16x2_scaled(v.z);
        hi.y = e4m3x2_to_f16x2_scaled(v.z >> 16);
        hi.z = e4m3x2_to_f16x2_scaled(v.w);
        hi.w = e4m3x2_to_f16x2_scaled(v.w >> 16);
        const uint32_t a0 = smem_tile + tile_off<D>(r, 2 * c);
        const uint32_t a1 = smem_tile + tile_off<D>(r, 2 * c + 1);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a0), "r"(lo.x), "r"(lo.y),
                     "r"(lo.z), "r"(lo.w) : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a1), "r"(hi.x), "r"(hi.y),
                     "r"(hi.z), "r"(hi.w) : "memory");
      }
    }
  }
};

// ------------------------------------------------------------------ split-KV kernel
// grid (Hkv, num_seqs, parts), 128 threads. MT = number of m16 query-row tiles.
//
// K and V tiles of 64 cached tokens stream into shared memory *as stored* (e4m3 bytes or
// bf16) through a multi-stage cp.async pipeline; nothing is staged in registers. For an e4m3
// cache the tensor-core fragments are widened to f16 when they are loaded:
//   * Q.K^T: ldmatrix on the raw bytes hands thread (g, t) four consecutive dims
//     4t..4t+3 of token g per 16-dim k step; the contraction index may be permuted freely as
//     long as both operands agree, so the Q fragments (kept in registers for the whole
//     kernel) are loaded with the same 4t.. ordering and no shuffle is needed.
//   * P.V: ldmatrix.trans on byte pairs hands thread (g, t) tokens 2t, 2t+1 of dims 2g and
//     2g+1; the even dims feed one n8 tile and the odd dims another, which only relabels
//     output columns (undone when O is written).
template <int ROWB>
__device__ __forceinline__ uint32_t raw_off(int row, int chunk) {
  return (uint32_t)(row * ROWB + ((chunk ^ (row & 7)) << 4));
}
// two e4m3 bytes -> f16x2 (exact). lo16 / hi16 take the low / high half of a 32-bit word,
// `sel` gathers an arbitrary byte pair first.
__device__ __forceinline__ uint32_t cvt_e4m3x2(uint16_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  return r;
}
__device__ __forceinline__ uint32_t e4m3_lo16(uint32_t x) { return cvt_e4m3x2((uint16_t)(x & 0xFFFFu)); }
__device__ __forceinline__ uint32_t e4m3_hi16(uint32_t x) { return cvt_e4m3x2((uint16_t)(x >> 16)); }
__device__ __forceinline__ uint32_t e4m3_sel(uint32_t x, uint32_t sel) {
  return cvt_e4m3x2((uint16_t)__byte_perm(x, 0, sel));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D, bool FP8, int MT>
struct SplitKvCfg {
  static constexpr int kRowB = FP8 ? D : 2 * D;                // bytes per cached row in smem
  static constexpr int kTileB = 64 * kRowB;                    // one K (or V) tile
  static constexpr int kStages = 3;
  static constexpr int kPipeB = kStages * 2 * kTileB;
  static constexpr int kMergeB = 4 * MT * 16 * 2 * 4 + 4 * MT * 16 * D * 4;
  static constexpr int kSmem = kPipeB > kMergeB ? kPipeB : kMergeB;
};

template <int D, bool FP8, int MT>
__global__ void __launch_bounds__(128, (D <= 128 && MT == 1) ? 4 : 1) attn_splitkv_kernel(const AttnParams p) {
  using C = SplitKvCfg<D, FP8, MT>;
  constexpr bool F16 = FP8;
  constexpr int kTile = 64;
  constexpr int kRowB = C::kRowB, kTileB = C::kTileB, kStages = C::kStages;
  constexpr int kChunks = kRowB / 16;                          // 16-byte chunks per row
  extern __shared__ __align__(128) uint8_t smem_attn[];
  const uint32_t sbase = mb::smem_u32(smem_attn);
  const int kvh = blockIdx.x, seq = blockIdx.y, part = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = p.Hq / p.Hkv;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int qlen = p.q_len[seq], ctx = p.ctx_len[seq], qs = p.q_start[seq];
  const int R = G * qlen;
  if (qlen <= 0) return;
  // partitions of one sequence: as many as a fixed partition size needs, then balanced
  // (a function of this sequence's own length only, never of the rest of the batch)
  const int nparts = max(1, (ctx + p.part_tokens - 1) / p.part_tokens);
  if (part >= nparts) return;
  const int part_len = (((ctx + nparts - 1) / nparts) + 63) & ~63;
  int tok_begin = part * part_len;
  const int tok_end = min(ctx, tok_begin + part_len);
  if (p.window > 0) tok_begin = max(tok_begin, (ctx - qlen + 1 - p.window) & ~63);
  if (tok_begin < 0) tok_begin = 0;
  const bool empty = tok_begin >= tok_end;
  const int* bt = p.block_table + (size_t)seq * p.max_blocks;
  const int ntiles = empty ? 0 : (tok_end - tok_begin + kTile - 1) / kTile;

  // block ids of this partition, staged once (bounds-checked here, not per chunk)
  constexpr int kMaxBlk = 160;                                 // 2496 tokens per partition at block 16
  __shared__ int s_blk[kMaxBlk];
  const int bs = p.block_size;
  const bool fast_blocks = (bs == 16 || bs == 32 || bs == 64) && (p.part_tokens + 64) / bs <= kMaxBlk;
  const int bs_shift = 31 - __clz(bs);
  if (!empty) {
    const int first_blk = tok_begin / bs, nblk = (tok_end - 1) / bs - first_blk + 1;
    for (int i = tid; i < nblk && i < kMaxBlk; i += 128) {
      int b = bt[first_blk + i];
      if (b < 0 || b >= p.num_blocks) {
        if (p.status) atomicCAS(p.status, 0u, MB_ST_BOUNDS);
        b = 0;
      }
      s_blk[i] = b;
    }
  }
  __syncthreads();
  // per-thread constants of the copy pattern: chunk i of a tile is row r_i, 16-byte column c_i
  constexpr int kCopies = (64 * kChunks) / 128;
  const size_t row_pitch = (size_t)p.Hkv * kRowB;              // bytes between consecutive tokens
  // When the rows a thread copies are a whole number of cache blocks apart, everything but the
  // block id is the same for every tile: one shared-memory read and one multiply-add per copy.
  constexpr int kStep = (kChunks <= 128 && 128 % kChunks == 0) ? 128 / kChunks : 0;   // rows between copies
  const bool lin = fast_blocks && kStep > 0 && (kStep % bs) == 0 && kCopies <= 8;
  const int r0 = tid / kChunks, c0 = tid % kChunks;
  const uint32_t soff0 = raw_off<kRowB>(r0, c0);               // kStep % 8 == 0: the swizzle term is fixed
  const size_t gbase = (size_t)(r0 & (bs - 1)) * row_pitch + (size_t)kvh * kRowB + (size_t)c0 * 16;
  const size_t blk_pitch = (size_t)bs * row_pitch;
  const int bsel0 = r0 >> bs_shift, bstep = kStep >> bs_shift;
  auto issue_tile = [&](int it) {
    const int stage = it % kStages;
    const uint32_t sK = sbase + stage * 2 * kTileB, sV = sK + kTileB;
    const int tok0 = tok_begin + it * kTile;
    const int blk0 = (tok0 - tok_begin) >> bs_shift;
    if (lin) {
#pragma unroll
      for (int i = 0; i < kCopies; ++i) {
        const bool valid = tok0 + r0 + i * kStep < tok_end;
        const int blk = valid ? s_blk[blk0 + bsel0 + i * bstep] : 0;
        const size_t off = (size_t)blk * blk_pitch + gbase;
        const int sz = valid ? 16 : 0;
        const uint32_t so = soff0 + (uint32_t)(i * kStep * kRowB);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sK + so),
                     "l"(reinterpret_cast<const uint8_t*>(p.k_cache) + off), "r"(sz) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sV + so),
                     "l"(reinterpret_cast<const uint8_t*>(p.v_cache) + off), "r"(sz) : "memory");
      }
      return;
    }
#pragma unroll
    for (int i = 0; i < kCopies; ++i) {
      const int idx = tid + i * 128;
      const int r = idx / kChunks, c = idx % kChunks;          // compile-time divisors
      const int tok = tok0 + r;
      int sz = 0;
      size_t off = 0;
      if (tok < tok_end) {
        int blk, within;
        if (fast_blocks) {
          blk = s_blk[blk0 + (r >> bs_shift)];
          within = r & (bs - 1);                                      // tiles start on a block boundary
        } else {
          blk = bt[tok / bs];
          within = tok % bs;
          if (blk < 0 || blk >= p.num_blocks) blk = 0;
        }
        off = ((size_t)blk * bs + within) * row_pitch + (size_t)kvh * kRowB + (size_t)c * 16;
        sz = 16;
      }
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sK + raw_off<kRowB>(r, c)),
                   "l"(reinterpret_cast<const uint8_t*>(p.k_cache) + off), "r"(sz) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sV + raw_off<kRowB>(r, c)),
                   "l"(reinterpret_cast<const uint8_t*>(p.v_cache) + off), "r"(sz) : "memory");
    }
  };

  // prologue: fill the pipeline, then load the Q fragments while the copies fly
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < ntiles) issue_tile(s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  uint32_t qf[MT][D / 16][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      const int r = mt * 16 + g + hr * 8;
      const __nv_bfloat16* qrow = nullptr;
      if (r < R) {
        const int tq = r / G, hh = r - tq * G;
        qrow = p.q + ((size_t)(qs + tq) * p.Hq + kvh * G + hh) * D;
      }
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t lo = 0, hi = 0;
        if (qrow) {
          if constexpr (FP8) {
            const uint2 v = *reinterpret_cast<const uint2*>(qrow + ks * 16 + 4 * t);
            const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
            const float2 f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
            lo = pack2<true>(f0.x, f0.y);
            hi = pack2<true>(f1.x, f1.y);
          } else {
            lo = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t);
            hi = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t + 8);
          }
        }
        qf[mt][ks][hr] = lo;          // a0 (row g) / a1 (row g + 8)
        qf[mt][ks][2 + hr] = hi;      // a2 / a3
      }
    }
  }

  // O accumulators: o_acc[mt][n][4]; for an e4m3 cache n = 2 * (16-dim group) + parity
  float o_acc[MT][D / 8][4];
  float m_run[MT][2], l_run[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) o_acc[mt][n][i] = 0.f;
  }
  const float kmul = FP8 ? (*p.k_scale) : 1.f;
  const float sc_log2 = p.scale * kmul * 1.44269504088896f;
  // rows of this thread: (mt, hr) -> causal limit; constant over the whole kernel
  int lim[MT][2];
  int min_limit = 0x7fffffff;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      const int r = mt * 16 + g + hr * 8;
      lim[mt][hr] = r < R ? ctx - qlen + r / G + 1 : 0x7fffffff;   // rows past R are never stored
      if (r < R) min_limit = min(min_limit, lim[mt][hr]);
    }
  min_limit = min(min_limit, __shfl_xor_sync(0xffffffffu, min_limit, 4));
  min_limit = min(min_limit, __shfl_xor_sync(0xffffffffu, min_limit, 8));
  min_limit = min(min_limit, __shfl_xor_sync(0xffffffffu, min_limit, 16));

  for (int it = 0; it < ntiles; ++it) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 2) : "memory");
    __syncthreads();
    if (it + kStages - 1 < ntiles) issue_tile(it + kStages - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const int stage = it % kStages;
    const uint32_t kT = sbase + stage * 2 * kTileB, vT = kT + kTileB;
    const int tok0 = tok_begin + it * kTile + warp * 16;
    if (tok0 >= tok_end) continue;
    float s[MT][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[mt][n][i] = 0.f;
    if constexpr (FP8) {
#pragma unroll
      for (int kg = 0; kg < D / 32; ++kg) {              // 32 dims = 2 k steps per ldmatrix.x4
        uint32_t r[4];
        // matrices: (tok 0-7, bytes lo) (tok 0-7, bytes hi) (tok 8-15, lo) (tok 8-15, hi)
        const int row = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
        ldsm4(r, kT + raw_off<kRowB>(row, kg * 2 + ((lane >> 3) & 1)));
#pragma unroll
        for (int h = 0; h < 2; ++h) {                     // k step 2 kg + h
          const uint32_t b00 = e4m3_lo16(r[h]), b01 = e4m3_hi16(r[h]);
          const uint32_t b10 = e4m3_lo16(r[2 + h]), b11 = e4m3_hi16(r[2 + h]);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma16816<true>(s[mt][0], qf[mt][kg * 2 + h], b00, b01);
            mma16816<true>(s[mt][1], qf[mt][kg * 2 + h], b10, b11);
          }
        }
      }
    } else {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t b[4];
        const int row = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
        ldsm4(b, kT + raw_off<kRowB>(row, ks * 2 + ((lane >> 3) & 1)));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma16816<false>(s[mt][0], qf[mt][ks], b[0], b[1]);
          mma16816<false>(s[mt][1], qf[mt][ks], b[2], b[3]);
        }
      }
    }
    // online softmax over this warp's 16 tokens; the mask code only runs for tiles that
    // touch a causal limit, the end of the range or a sliding window
    const bool need_mask = (tok0 + 16 > min_limit) || (tok0 + 16 > tok_end) || (p.window > 0);
    uint32_t pa[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int hr = 0; hr < 2; ++hr) {
        float mx = -INFINITY;
        if (need_mask) {
          const int limit = min(lim[mt][hr], tok_end);
          const int wlo = p.window > 0 ? lim[mt][hr] - p.window : 0;
#pragma unroll
          for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const int tok = tok0 + n * 8 + t * 2 + i;
              float v = s[mt][n][hr * 2 + i] * sc_log2;
              if (tok >= limit || tok < wlo) v = -INFINITY;
              s[mt][n][hr * 2 + i] = v;
              mx = fmaxf(mx, v);
            }
        } else {
#pragma unroll
          for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const float v = s[mt][n][hr * 2 + i] * sc_log2;
              s[mt][n][hr * 2 + i] = v;
              mx = fmaxf(mx, v);
            }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[mt][hr], mx);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = fast_exp2(m_run[mt][hr] - m_use);
        float rs = 0.f;
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const float pv = fast_exp2(s[mt][n][hr * 2 + i] - m_use);
            s[mt][n][hr * 2 + i] = pv;
            rs += pv;
          }
        l_run[mt][hr] = l_run[mt][hr] * alpha + rs;
        m_run[mt][hr] = m_new;
        if (alpha != 1.f) {
#pragma unroll
          for (int n = 0; n < D / 8; ++n) {
            o_acc[mt][n][hr * 2] *= alpha;
            o_acc[mt][n][hr * 2 + 1] *= alpha;
          }
        }
      }
      pa[mt][0] = pack2<F16>(s[mt][0][0], s[mt][0][1]);
      pa[mt][1] = pack2<F16>(s[mt][0][2], s[mt][0][3]);
      pa[mt][2] = pack2<F16>(s[mt][1][0], s[mt][1][1]);
      pa[mt][3] = pack2<F16>(s[mt][1][2], s[mt][1][3]);
    }
    // O += P V
    if constexpr (FP8) {
#pragma unroll
      for (int d2 = 0; d2 < D / 32; ++d2) {               // two 16-dim groups per ldmatrix.x4.trans
        uint32_t r[4];
        // matrices: (tok 0-7, grp 2 d2) (tok 8-15, grp 2 d2) (tok 0-7, grp 2 d2 + 1) (tok 8-15, ...)
        const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        ldsm4t(r, vT + raw_off<kRowB>(row, d2 * 2 + (lane >> 4)));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int dg = d2 * 2 + h;
          const uint32_t e0 = e4m3_sel(r[2 * h], 0x4420), e1 = e4m3_sel(r[2 * h + 1], 0x4420);
          const uint32_t o0 = e4m3_sel(r[2 * h], 0x4431), o1 = e4m3_sel(r[2 * h + 1], 0x4431);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma16816<true>(o_acc[mt][dg * 2], pa[mt], e0, e1);        // even dims of the group
            mma16816<true>(o_acc[mt][dg * 2 + 1], pa[mt], o0, o1);    // odd dims
          }
        }
      }
    } else {
#pragma unroll
      for (int n2 = 0; n2 < D / 16; ++n2) {
        uint32_t b[4];
        const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        ldsm4t(b, vT + raw_off<kRowB>(row, n2 * 2 + (lane >> 4)));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma16816<false>(o_acc[mt][n2 * 2], pa[mt], b[0], b[1]);
          mma16816<false>(o_acc[mt][n2 * 2 + 1], pa[mt], b[2], b[3]);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  // ---- merge the 4 warps through shared memory (the pipeline buffers are free now)
  float* s_ml = reinterpret_cast<float*>(smem_attn);
  float* s_o = s_ml + 4 * MT * 16 * 2;
  const float vmul = FP8 ? (*p.v_scale) : 1.f;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      const int r = mt * 16 + g + hr * 8;
      float l = l_run[mt][hr];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if (t == 0) {
        s_ml[(warp * MT * 16 + r) * 2] = m_run[mt][hr];
        s_ml[(warp * MT * 16 + r) * 2 + 1] = l;
      }
      float* orow = s_o + ((size_t)(warp * MT * 16 + r)) * D;
      if constexpr (FP8) {
#pragma unroll
        for (int dg = 0; dg < D / 16; ++dg) {
          // even tile cols (2t, 2t+1) -> dims 4t, 4t+2 ; odd tile -> dims 4t+1, 4t+3
          float4 v4;
          v4.x = o_acc[mt][dg * 2][hr * 2];
          v4.y = o_acc[mt][dg * 2 + 1][hr * 2];
          v4.z = o_acc[mt][dg * 2][hr * 2 + 1];
          v4.w = o_acc[mt][dg * 2 + 1][hr * 2 + 1];
          *reinterpret_cast<float4*>(orow + dg * 16 + 4 * t) = v4;
        }
      } else {
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
          orow[n * 8 + t * 2] = o_acc[mt][n][hr * 2];
          orow[n * 8 + t * 2 + 1] = o_acc[mt][n][hr * 2 + 1];
        }
      }
    }
  __syncthreads();
  for (int idx = tid; idx < R * (D / 4); idx += 128) {
    const int r = idx / (D / 4), c4 = idx - r * (D / 4);
    float mw[4], lw[4];
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      mw[w] = s_ml[(w * MT * 16 + r) * 2];
      lw[w] = s_ml[(w * MT * 16 + r) * 2 + 1];
      mx = fmaxf(mx, mw[w]);
    }
    float l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = mw[w] == -INFINITY ? 0.f : exp2f(mw[w] - mx);
      l += lw[w] * f;
      const float4 ov = *reinterpret_cast<const float4*>(s_o + ((size_t)(w * MT * 16 + r)) * D + c4 * 4);
      acc.x += ov.x * f; acc.y += ov.y * f; acc.z += ov.z * f; acc.w += ov.w * f;
    }
    const float inv = l > 0.f ? vmul / l : 0.f;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    const int tq = r / G, hh = r - tq * G;
    const size_t orow = (size_t)(qs + tq) * p.Hq + kvh * G + hh;
    if (nparts == 1) {
      store_out4<D>(p, orow, c4, acc.x, acc.y, acc.z, acc.w);
    } else {
      *reinterpret_cast<float4*>(p.part_o + (orow * p.parts + part) * D + c4 * 4) = acc;
      if (c4 == 0) {
        p.part_ml[(orow * p.parts + part) * 2] = mx;          // log2-domain max
        p.part_ml[(orow * p.parts + part) * 2 + 1] = l;
      }
    }
  }
  if (nparts == 1) return;
  // the last partition of this (sequence, kv head) to arrive merges all of them, in
  // partition order, and re-arms the counter
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const uint32_t prev = atomicAdd(&p.part_cnt[seq * p.Hkv + kvh], 1u);
    s_last = (prev == (uint32_t)nparts - 1);
    if (s_last) p.part_cnt[seq * p.Hkv + kvh] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = tid; idx < R * (D / 4); idx += 128) {
    const int r = idx / (D / 4), c4 = idx - r * (D / 4);
    const int tq = r / G, hh = r - tq * G;
    const size_t orow = (size_t)(qs + tq) * p.Hq + kvh * G + hh;
    float mx = -INFINITY;
    for (int s2 = 0; s2 < nparts; ++s2) mx = fmaxf(mx, __ldcg(&p.part_ml[(orow * p.parts + s2) * 2]));
    float denom = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s2 = 0; s2 < nparts; ++s2) {
      const float m = __ldcg(&p.part_ml[(orow * p.parts + s2) * 2]);
      const float l = __ldcg(&p.part_ml[(orow * p.parts + s2) * 2 + 1]);
      if (m == -INFINITY || l <= 0.f) continue;
      const float wgt = l * exp2f(m - mx);
      denom += wgt;
      const float4 ov = __ldcg(reinterpret_cast<const float4*>(p.part_o + (orow * p.parts + s2) * D + c4 * 4));
      acc.x += ov.x * wgt; acc.y += ov.y * wgt; acc.z += ov.z * wgt; acc.w += ov.w * wgt;
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    store_out4<D>(p, orow, c4, acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
  }
}

// ------------------------------------------------------------------ split-Q (prefill) kernel
// grid (ceil(max_q_len / 64), Hq, num_seqs), 128 threads; warp w owns query rows 16w..16w+15.
template <int D, bool FP8>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const AttnParams p) {
  constexpr bool F16 = FP8;
  constexpr int kTile = 64;
  constexpr int kTileBytes = kTile * D * 2;
  extern __shared__ __align__(128) uint8_t smem_attn[];
  const uint32_t sbase = mb::smem_u32(smem_attn);
  const uint32_t sQ = sbase;
  const uint32_t sK = sbase + kTileBytes;
  const uint32_t sV = sK + 2 * kTileBytes;
  const int qt = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.Hq / p.Hkv, kvh = head / G;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int qlen = p.q_len[seq], ctx = p.ctx_len[seq], qs = p.q_start[seq];
  const int q0 = qt * 64;
  if (q0 >= qlen) return;
  const int* bt = p.block_table + (size_t)seq * p.max_blocks;
  const int past = ctx - qlen;                                 // tokens cached before this chunk
  const int tok_end = min(ctx, past + q0 + 64);                // causal upper bound for the tile
  int tok_begin = 0;
  if (p.window > 0) tok_begin = max(0, past + q0 + 1 - p.window);
  tok_begin &= ~63;

  for (int idx = tid; idx < 64 * (D / 8); idx += 128) {
    const int r = idx / (D / 8), c = idx - r * (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (q0 + r < qlen) {
      v = *reinterpret_cast<const uint4*>(p.q + ((size_t)(qs + q0 + r) * p.Hq + head) * D + c * 8);
      if constexpr (F16) {
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
        uint4 o;
        uint32_t* oo = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(b[i]);
          oo[i] = pack2<true>(f.x, f.y);
        }
        v = o;
      }
    }
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(sQ + tile_off<D>(r, c)), "r"(v.x),
                 "r"(v.y), "r"(v.z), "r"(v.w));
  }

  float o_acc[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[n][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float kmul = FP8 ? (*p.k_scale) * 256.f : 1.f;
  const float sc_log2 = p.scale * kmul * 1.44269504088896f;

  TileLoader<D, FP8> ldK, ldV;
  const int ntiles = (tok_end - tok_begin + kTile - 1) / kTile;
  ldK.fetch(p, p.k_cache, bt, kvh, tok_begin, tok_end, tid, sK);
  ldV.fetch(p, p.v_cache, bt, kvh, tok_begin, tok_end, tid, sV);
  for (int it = 0; it < ntiles; ++it) {
    const int buf = it & 1;
    ldK.commit(sK + buf * kTileBytes, tid);
    ldV.commit(sV + buf * kTileBytes, tid);
    __syncthreads();
    if (it + 1 < ntiles) {
      ldK.fetch(p, p.k_cache, bt, kvh, tok_begin + (it + 1) * kTile, tok_end, tid,
                sK + (buf ^ 1) * kTileBytes);
      ldV.fetch(p, p.v_cache, bt, kvh, tok_begin + (it + 1) * kTile, tok_end, tid,
                sV + (buf ^ 1) * kTileBytes);
    }
    const uint32_t kT = sK + buf * kTileBytes, vT = sV + buf * kTileBytes;
    const int tile_tok0 = tok_begin + it * kTile;
    // S[16 x 64] for this warp
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      ldsm4(a, sQ + tile_off<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        uint32_t b[4];
        const int row = nb * 16 + (lane & 7) + ((lane >> 4) << 3);
        ldsm4(b, kT + tile_off<D>(row, ks * 2 + ((lane >> 3) & 1)));
        mma16816<F16>(s[nb * 2], a, b[0], b[1]);
        mma16816<F16>(s[nb * 2 + 1], a, b[2], b[3]);
      }
    }
    float alpha[2];
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      const int qr = q0 + warp * 16 + (lane >> 2) + hr * 8;    // query index inside the chunk
      const int limit = past + qr + 1;
      const int wlo = p.window > 0 ? limit - p.window : 0;
      float mx = -INFINITY;
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int tok = tile_tok0 + n * 8 + (lane & 3) * 2 + i;
          float v = s[n][hr * 2 + i] * sc_log2;
          if (tok >= limit || tok >= tok_end || tok < wlo || qr >= qlen) v = -INFINITY;
          s[n][hr * 2 + i] = v;
          mx = fmaxf(mx, v);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[hr], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      alpha[hr] = exp2f(m_run[hr] - m_use);
      float rs = 0.f;
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float pv = exp2f(s[n][hr * 2 + i] - m_use);
          s[n][hr * 2 + i] = pv;
          rs += pv;
        }
      l_run[hr] = l_run[hr] * alpha[hr] + rs;
      m_run[hr] = m_new;
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      o_acc[n][0] *= alpha[0]; o_acc[n][1] *= alpha[0];
      o_acc[n][2] *= alpha[1]; o_acc[n][3] *= alpha[1];
    }
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {                            // 16 tokens per k step
      uint32_t pa[4];
      pa[0] = pack2<F16>(s[kb * 2][0], s[kb * 2][1]);
      pa[1] = pack2<F16>(s[kb * 2][2], s[kb * 2][3]);
      pa[2] = pack2<F16>(s[kb * 2 + 1][0], s[kb * 2 + 1][1]);
      pa[3] = pack2<F16>(s[kb * 2 + 1][2], s[kb * 2 + 1][3]);
#pragma unroll
      for (int n2 = 0; n2 < D / 16; ++n2) {
        uint32_t b[4];
        const int row = kb * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        ldsm4t(b, vT + tile_off<D>(row, n2 * 2 + (lane >> 4)));
        mma16816<F16>(o_acc[n2 * 2], pa, b[0], b[1]);
        mma16816<F16>(o_acc[n2 * 2 + 1], pa, b[2], b[3]);
      }
    }
    __syncthreads();
  }
  const float vmul = FP8 ? (*p.v_scale) * 256.f : 1.f;
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    float l = l_run[hr];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int qr = q0 + warp * 16 + (lane >> 2) + hr * 8;
    if (qr >= qlen) continue;
    const float inv = l > 0.f ? vmul / l : 0.f;
    __nv_bfloat16* dst = p.out + ((size_t)(qs + qr) * p.Hq + head) * D + (lane & 3) * 2;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
      *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) =
          __floats2bfloat162_rn(o_acc[n][hr * 2] * inv, o_acc[n][hr * 2 + 1] * inv);
  }
}

template <int D, bool FP8, int MT>
int launch_splitkv(const AttnParams& p, int num_seqs, cudaStream_t stream) {
  constexpr int smem = SplitKvCfg<D, FP8, MT>::kSmem;
  auto kern = attn_splitkv_kernel<D, FP8, MT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)mb::launch_kernel(kern, dim3(p.Hkv, num_seqs, p.parts), dim3(128), smem, stream, p);
}
template <int D, bool FP8>
int launch_prefill(const AttnParams& p, int num_seqs, int max_q_len, cudaStream_t stream) {
  constexpr int smem = 5 * 64 * D * 2;
  auto kern = attn_prefill_kernel<D, FP8>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)mb::launch_kernel(kern, dim3((max_q_len + 63) / 64, p.Hq, num_seqs), dim3(128), smem, stream, p);
}

template <int D, bool FP8>
int dispatch_mt(int mt, const AttnParams& p, int num_seqs, cudaStream_t stream) {
  if (mt == 1) return launch_splitkv<D, FP8, 1>(p, num_seqs, stream);
  // two m16 row tiles keep 2 * D / 2 accumulator registers per thread: fits up to D = 128
  if constexpr (D <= 128) {
    if (mt == 2) return launch_splitkv<D, FP8, 2>(p, num_seqs, stream);
  }
  return MB_ERR_UNSUPPORTED;
}

}  // namespace

extern "C" {

struct MbRopeKvArgs {
  int M, Hq, Hkv, D, rot;
  const void* qkv;
  long long qkv_ld;
  int q_head_stride, k_off, v_off;
  const int* positions;
  const long long* slots;
  const void* q_norm_w;
  const void* k_norm_w;
  int norm_plus_one;
  float eps;
  const float* cos_tab;
  const float* sin_tab;
  int max_pos;
  void* q_out;
  void* k_cache;
  void* v_cache;
  int cache_fp8;
  const float* k_scale;
  const float* v_scale;
  long long num_slots;
  uint32_t* status;
  float* amax;             // optional [2] running max |k|, |v| of the written rows
};

// value * old_scale / *new_scale for every listed slot of an e4m3 cache [num_slots, row_elems]
int mb_kv_rescale(void* cache, const long long* slots, int n, int row_elems, long long num_slots, float old_scale,
                  const float* new_scale, cudaStream_t stream) {
  if (!cache || !slots || !new_scale || n <= 0 || row_elems <= 0 || !(old_scale > 0.f)) return MB_ERR_BAD_ARG;
  kv_rescale_kernel<<<n, 256, 0, stream>>>(reinterpret_cast<uint8_t*>(cache), slots, n, row_elems, num_slots, old_scale,
                                           new_scale);
  return (int)cudaGetLastError();
}

int mb_qk_norm_rope_kvwrite(const MbRopeKvArgs* a, cudaStream_t stream) {
  if (!a || a->M <= 0 || !a->qkv || !a->q_out || !a->slots) return MB_ERR_BAD_ARG;
  if (a->D % 32 || a->D > 256) return MB_ERR_UNSUPPORTED;
  if (a->cos_tab && ((a->rot % 64 && a->rot != 32) || a->rot > a->D || !a->positions)) return MB_ERR_UNSUPPORTED;
  if (a->cache_fp8 && (!a->k_scale || !a->v_scale)) return MB_ERR_BAD_ARG;
  RopeKvParams p{};
  p.M = a->M; p.Hq = a->Hq; p.Hkv = a->Hkv; p.D = a->D; p.rot = a->rot;
  p.qkv = reinterpret_cast<const __nv_bfloat16*>(a->qkv); p.qkv_ld = a->qkv_ld;
  p.q_head_stride = a->q_head_stride; p.k_off = a->k_off; p.v_off = a->v_off;
  p.positions = a->positions; p.slots = a->slots;
  p.q_norm_w = reinterpret_cast<const __nv_bfloat16*>(a->q_norm_w);
  p.k_norm_w = reinterpret_cast<const __nv_bfloat16*>(a->k_norm_w);
  p.norm_plus_one = a->norm_plus_one; p.eps = a->eps;
  p.cos_tab = a->cos_tab; p.sin_tab = a->sin_tab; p.max_pos = a->max_pos;
  p.q_out = reinterpret_cast<__nv_bfloat16*>(a->q_out);
  p.k_cache = a->k_cache; p.v_cache = a->v_cache; p.cache_fp8 = a->cache_fp8;
  p.k_scale = a->k_scale; p.v_scale = a->v_scale; p.num_slots = a->num_slots;
  p.status = a->status;
  p.amax = a->amax;
  const int Htot = a->Hq + 2 * a->Hkv;
  return (int)mb::launch_kernel(rope_kv_kernel, dim3(a->M, (Htot + 3) / 4), dim3(128), 0, stream, p);
}

struct MbAttnArgs {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const int* block_table;
  int max_blocks;
  const int* q_start;
  const int* q_len;
  const int* ctx_len;
  int num_seqs, max_q_len, max_ctx;
  int Hq, Hkv, D, block_size;
  long long num_blocks;
  float scale;
  int cache_fp8;
  const float* k_scale;
  const float* v_scale;
  void* out;
  void* ws;                // split-KV partials
  size_t ws_bytes;
  int total_rows;          // query rows (for workspace sizing)
  int part_tokens;         // 0 = default 512
  int window;
  int force_mode;          // 0 auto, 1 split-KV, 2 split-Q
  uint32_t* status;
  void* outq;              // optional NVFP4 output (split-KV path only; MB_ERR_UNSUPPORTED otherwise)
  int ldq;
  void* outq_sf;
  int outq_sf_k64;
  float outq_gs;
};

// workspace bytes for the split-KV path
size_t mb_attn_ws_bytes(int total_rows, int Hq, int D, int max_ctx, int part_tokens) {
  const int pt = part_tokens > 0 ? part_tokens : 512;
  const int parts = (max_ctx + pt - 1) / pt;
  if (parts <= 1) return 0;
  return kAttnCntBytes + (size_t)total_rows * Hq * parts * (D + 2) * sizeof(float);
}

int mb_paged_attention(const MbAttnArgs* a, cudaStream_t stream) {
  if (!a || !a->q || !a->k_cache || !a->v_cache || !a->block_table || !a->out) return MB_ERR_BAD_ARG;
  if (a->num_seqs <= 0 || a->Hkv <= 0 || a->Hq % a->Hkv) return MB_ERR_BAD_ARG;
  if (a->cache_fp8 && (!a->k_scale || !a->v_scale)) return MB_ERR_BAD_ARG;
  AttnParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(a->q);
  p.k_cache = a->k_cache; p.v_cache = a->v_cache;
  p.block_table = a->block_table; p.max_blocks = a->max_blocks;
  p.q_start = a->q_start; p.q_len = a->q_len; p.ctx_len = a->ctx_len;
  p.Hq = a->Hq; p.Hkv = a->Hkv; p.block_size = a->block_size; p.num_blocks = a->num_blocks;
  p.scale = a->scale; p.k_scale = a->k_scale; p.v_scale = a->v_scale;
  p.out = reinterpret_cast<__nv_bfloat16*>(a->out);
  p.window = a->window; p.status = a->status;
  const int G = a->Hq / a->Hkv;
  const int rows = G * a->max_q_len;
  int mode = a->force_mode;
  if (mode == 0) mode = rows <= 32 ? 1 : 2;
  const bool fp8 = a->cache_fp8 != 0;
  if (a->outq) {
    if (mode != 1 || a->D % 128 || !a->outq_sf || a->outq_gs <= 0.f || a->outq_sf_k64 * 64 < a->Hq * a->D)
      return MB_ERR_UNSUPPORTED;
    p.outq = reinterpret_cast<uint8_t*>(a->outq); p.ldq = a->ldq;
    p.outq_sf = reinterpret_cast<uint8_t*>(a->outq_sf); p.outq_sf_k64 = a->outq_sf_k64;
    p.outq_gs = a->outq_gs;
  }
  if (mode == 1) {
    if (rows > 32) return MB_ERR_UNSUPPORTED;
    const int mt = rows <= 16 ? 1 : 2;
    p.part_tokens = a->part_tokens > 0 ? a->part_tokens : 512;
    p.parts = (a->max_ctx + p.part_tokens - 1) / p.part_tokens;
    if (p.parts < 1) p.parts = 1;
    if (p.parts > 1) {
      const size_t cnt_bytes = ((size_t)a->num_seqs * a->Hkv * sizeof(uint32_t) + 255) & ~size_t(255);
      const size_t need = cnt_bytes + (size_t)a->total_rows * a->Hq * p.parts * (a->D + 2) * sizeof(float);
      if (!a->ws || a->ws_bytes < need || cnt_bytes > kAttnCntBytes) return MB_ERR_TOO_LARGE;
      // counters sit in the first kAttnCntBytes of the workspace (zero-initialised by the
      // owner once; every launch leaves them at zero again)
      p.part_cnt = reinterpret_cast<uint32_t*>(a->ws);
      p.part_o = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a->ws) + kAttnCntBytes);
      p.part_ml = p.part_o + (size_t)a->total_rows * a->Hq * p.parts * a->D;
    }
    int rc;
    if (a->D == 128) rc = fp8 ? dispatch_mt<128, true>(mt, p, a->num_seqs, stream)
                              : dispatch_mt<128, false>(mt, p, a->num_seqs, stream);
    else if (a->D == 64) rc = fp8 ? dispatch_mt<64, true>(mt, p, a->num_seqs, stream)
                                  : dispatch_mt<64, false>(mt, p, a->num_seqs, stream);
    else if (a->D == 256) rc = fp8 ? dispatch_mt<256, true>(mt, p, a->num_seqs, stream)
                                   : dispatch_mt<256, false>(mt, p, a->num_seqs, stream);
    else return MB_ERR_UNSUPPORTED;
    return rc;                    // partitions are merged inside the kernel by the last arriver
  }
  p.parts = 1;
  if (a->D == 128) return fp8 ? launch_prefill<128, true>(p, a->num_seqs, a->max_q_len, stream)
                              : launch_prefill<128, false>(p, a->num_seqs, a->max_q_len, stream);
  if (a->D == 64) return fp8 ? launch_prefill<64, true>(p, a->num_seqs, a->max_q_len, stream)
                             : launch_prefill<64, false>(p, a->num_seqs, a->max_q_len, stream);
  if (a->D == 256) return fp8 ? launch_prefill<256, true>(p, a->num_seqs, a->max_q_len, stream)
                              : launch_prefill<256, false>(p, a->num_seqs, a->max_q_len, stream);
  return MB_ERR_UNSUPPORTED;
}

}  // extern "C"
