// Prefill attention on the 5th-generation tensor cores: both products of a 128-query-row tile run
// as tcgen05.mma with the accumulators in tensor memory.
//
// One CTA = 128 query rows of one query head of one sequence (grid: q tiles x heads x sequences),
// 128 threads, thread r owns query row r. Per tile of 64 cached tokens:
//   1. all threads stage the K tile ([64 tokens x 128 dims], K-major, two 64-dim halves) and the
//      transposed V tile ([128 dims x 64 tokens], K-major in the token direction) into shared memory
//      in the 128-byte-swizzled layout the matrix descriptors describe; an e4m3 cache is widened
//      to bf16 on the way (exactly; its 2^-8 shift and the cache scales fold into the softmax scale
//      and the final normalisation);
//   2. one thread issues S = Q K^T (M 128, N 64, eight k steps of 16) into TMEM columns 0..63 and
//      commits to an mbarrier;
//   3. every thread reads its row of S back with tcgen05.ld, applies scale, causal limit and the
//      online-softmax update (row maximum and sum live in the thread: no shuffles), and writes its
//      row of P as bf16 into the swizzled P tile;
//   4. one thread issues O_j = P V (M 128, N 128, four k steps) into TMEM columns 64..191;
//   5. every thread folds its row of O_j into its fp32 output row in registers
//      (o = o * alpha + O_j), so the rescale is exact on every tile.
// Two CTAs fit an SM (80 KB of shared memory, 256 TMEM columns each), so one CTA's staging and
// softmax overlap the other's tensor work. Every wait on an mbarrier is bounded and reports
// through the status word; TMEM is freed on every path.
//
// Serves q_len >= 128 chunks with head_dim 128, bf16 or e4m3 caches, no sliding window; other
// shapes stay on the mma.sync kernels in attention.cu, which are also the oracle in the tests.
// Reference behaviour covered: the prefill paged-attention family
// (kernels/gb10/common/prefill_paged_compute.cuh:3-7,37-41), re-designed for TMEM accumulators.
#include "common.cuh"

namespace {

constexpr int kQ = 128;          // query rows per CTA
constexpr int kT = 64;           // cached tokens per tile
constexpr int kHalfB = 64 * 2;   // bytes of a 64-element bf16 swizzle row

struct TcParams {
  const __nv_bfloat16* q;        // [rows, Hq, D]
  const void* k_cache;           // [blocks, block, Hkv, D] bf16 or e4m3
  const void* v_cache;
  const int* block_table;
  int max_blocks;
  const int* q_start;
  const int* q_len;
  const int* ctx_len;
  int Hq, Hkv, block_size;
  long long num_blocks;
  float scale;
  const float* k_scale;
  const float* v_scale;
  __nv_bfloat16* out;            // [rows, Hq, D]
  uint32_t* status;
};

// byte offset of 16-byte chunk `c` of row `r` in a tile of 128-byte rows with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw_off(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// eight e4m3 bytes -> eight bf16 holding value * 2^-8 (exact, denormals included)
__device__ __forceinline__ uint4 widen8(uint2 v) {
  uint4 o;
  uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t word = i < 2 ? v.x : v.y;
    const uint32_t two = (i & 1) ? (word >> 16) : word;
    const uint32_t w = __byte_perm(two, 0, 0x1404);                        // b0 -> bits 15:8, b1 -> bits 31:24
    const uint32_t h = (w & 0x80008000u) | ((w & 0x7F007F00u) >> 1);       // f16x2 = value * 2^-8
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
    const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
    ow[i] = *reinterpret_cast<const uint32_t*>(&b);
  }
  return o;
}

// kD = head dim (128 or 256; 256 needs the MN-major V path). kNH = 64-dim blocks per row; a staging
// thread owns one token and the blocks sub, sub + 2, ... (sub = tid / 64).
template <int kD, bool FP8, bool VMN>
__global__ void __launch_bounds__(128, kD == 128 ? 2 : 1) attn_prefill_tc_kernel(const TcParams p) {
  static_assert(kD == 128 || (kD == 256 && VMN), "head dim 256 stages V as stored");
  constexpr int kNH = kD / 64, kNHT = kNH / 2;
  constexpr uint32_t kTmemCols = kD == 128 ? 256 : 512;    // S (64) + O (kD), rounded to a power of two
  extern __shared__ __align__(16) uint8_t smem[];
  // the swizzled tiles need 1024-byte alignment in the shared window (the launch reserves the slack)
  uint8_t* sQ = smem + ((1024u - (mb::smem_u32(smem) & 1023u)) & 1023u);   // kNH blocks x [128 rows x 128 B]
  uint8_t* sK = sQ + kNH * kQ * 128;        // kNH blocks x [64 rows x 128 B]
  uint8_t* sV = sK + kNH * kT * 128;        // as stored: kNH blocks x [64 tokens x 128 B]; transposed: [kD dims x 128 B]
  uint8_t* sP = sV + kD * 128;              // [128 rows x 128 B (64 tokens)]
  __shared__ uint64_t bar_s, bar_o;
  __shared__ uint32_t s_tmem;
  const int qt = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5;
  mb::pdl_wait();
  const int qlen = p.q_len[seq], ctx = p.ctx_len[seq], qs = p.q_start[seq];
  const int q0 = qt * kQ;
  if (q0 >= qlen) return;
  const int kvh = head / (p.Hq / p.Hkv);
  const int* bt = p.block_table + (size_t)seq * p.max_blocks;
  if (tid == 0) {
    mb::mbar_init(&bar_s, 1);
    mb::mbar_init(&bar_o, 1);
    mb::mbar_fence_init();
  }
  if (warp == 0) mb::tmem_alloc(&s_tmem, kTmemCols);
  // Q tile: thread = row
  {
    const int qi = q0 + tid;
    const uint4* src = qi < qlen ? reinterpret_cast<const uint4*>(p.q + ((size_t)(qs + qi) * p.Hq + head) * kD) : nullptr;
#pragma unroll
    for (int c = 0; c < kD / 8; ++c) {
      const uint4 v = src ? src[c] : make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(sQ + (c >> 3) * (kQ * 128) + sw_off(tid, c & 7)) = v;
    }
  }
  mb::tc_fence_before();
  __syncthreads();
  mb::tc_fence_after();
  // only now may a dependent kernel start early on this SM: it would allocate TMEM before its own
  // dependency wait, and must not do so while this CTA still has to get its columns
  mb::pdl_launch_dependents();
  const uint32_t tmem = s_tmem;
  const uint32_t t_row = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's 32 TMEM lanes
  constexpr uint32_t kIdescS = mb::umma_idesc(1, 1, kQ, kT);
  constexpr uint32_t kIdescO = mb::umma_idesc(1, 1, kQ, kD, 0, VMN ? 1 : 0);
  const uint32_t aQ = mb::smem_u32(sQ), aK = mb::smem_u32(sK), aV = mb::smem_u32(sV), aP = mb::smem_u32(sP);

  const int qi = q0 + tid;
  const bool row_ok = qi < qlen;
  const int limit = row_ok ? ctx - qlen + qi + 1 : 0;                // tokens [0, limit) are visible
  const int first_limit = (qlen - q0 >= kQ) ? ctx - qlen + q0 + 1 : 0;  // smallest limit of the CTA's rows (0: ragged tile, always mask)
  const int last_row = min(qlen, q0 + kQ) - 1;
  const int tiles = (ctx - qlen + last_row + 1 + kT - 1) / kT;        // up to the last row's limit
  const float kmul = FP8 ? (*p.k_scale) * 256.f : 1.f;
  const float sc_log2 = p.scale * kmul * 1.44269504088896f;
  float m_run = -INFINITY, l_run = 0.f;
  uint32_t ph_s = 0, ph_o = 0;
  bool ok = true;
  const size_t esz = FP8 ? 1 : 2;
  const size_t row_pitch = (size_t)p.Hkv * kD * esz;
  const int s_tok = tid & 63, s_half = tid >> 6;                      // staging: one token, one 64-dim half
  // raw cache bytes of this thread's token (blocks sub, sub + 2, ...) of the next tile, fetched one tile ahead
  constexpr int kRaw = FP8 ? 4 : 8;
  uint4 kraw[kNHT][kRaw], vraw[kNHT][kRaw];
  auto fetch = [&](int jt) {
    const int tok = jt * kT + s_tok;
    if (jt < tiles && tok < ctx) {
      long long blk = bt[tok / p.block_size];
      if (blk < 0 || blk >= p.num_blocks) {
        if (p.status) atomicCAS(p.status, 0u, MB_ST_BOUNDS);
        blk = 0;
      }
      const size_t off = ((size_t)blk * p.block_size + (tok % p.block_size)) * row_pitch + (size_t)kvh * kD * esz;
#pragma unroll
      for (int hh = 0; hh < kNHT; ++hh) {
        const size_t o2 = off + (size_t)(s_half + 2 * hh) * 64 * esz;
        const uint4* ks = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.k_cache) + o2);
        const uint4* vs = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.v_cache) + o2);
#pragma unroll
        for (int c = 0; c < kRaw; ++c) {
          kraw[hh][c] = __ldg(ks + c);
          vraw[hh][c] = __ldg(vs + c);
        }
      }
    } else {
#pragma unroll
      for (int hh = 0; hh < kNHT; ++hh)
#pragma unroll
        for (int c = 0; c < kRaw; ++c) kraw[hh][c] = vraw[hh][c] = make_uint4(0, 0, 0, 0);
    }
  };
  fetch(0);

  for (int j = 0; j < tiles; ++j) {
    // ---- the previous tile's P V has to be done before its operands are overwritten (and O read)
    if (j > 0) {
      ok = mb::mbar_wait(&bar_o, ph_o, p.status, MB_ST_TIMEOUT_MMA) && ok;
      ph_o ^= 1;
      mb::tc_fence_after();
    }
    // ---- stage K (K-major) and V (transposed) of tokens [j * 64, j * 64 + 64) from the registers
#pragma unroll
    for (int hh = 0; hh < kNHT; ++hh) {
      const int blk64 = s_half + 2 * hh;                 // which 64-dim block of the row
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 kv, vv;
        if constexpr (FP8) {
          const uint32_t* kw = reinterpret_cast<const uint32_t*>(&kraw[hh][c >> 1]);
          const uint32_t* vw = reinterpret_cast<const uint32_t*>(&vraw[hh][c >> 1]);
          kv = widen8(make_uint2(kw[(c & 1) * 2], kw[(c & 1) * 2 + 1]));
          vv = widen8(make_uint2(vw[(c & 1) * 2], vw[(c & 1) * 2 + 1]));
        } else {
          kv = kraw[hh][c];
          vv = vraw[hh][c];
        }
        *reinterpret_cast<uint4*>(sK + blk64 * (kT * 128) + sw_off(s_tok, c)) = kv;
        if constexpr (VMN) {
          // V as stored, [token][dim] in 64-dim blocks: read by the second product as an MN-major operand
          *reinterpret_cast<uint4*>(sV + blk64 * (kT * 128) + sw_off(s_tok, c)) = vv;
        } else {
          // V^T: element (dim d, token t) at row d, byte 2 t (chunk t / 8)
          const uint16_t* e = reinterpret_cast<const uint16_t*>(&vv);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int d = blk64 * 64 + c * 8 + i;
            *reinterpret_cast<uint16_t*>(sV + sw_off(d, s_tok >> 3) + (s_tok & 7) * 2) = e[i];
          }
        }
      }
    }
    fence_async_smem();
    mb::tc_fence_before();
    __syncthreads();
    // ---- S = Q K^T
    if (tid == 0) {
      mb::tc_fence_after();
#pragma unroll
      for (int h = 0; h < kNH; ++h)
#pragma unroll
        for (int s = 0; s < 4; ++s)
          mb::umma_f16(tmem, mb::umma_desc_sw128(aQ + h * (kQ * 128) + s * 32),
                       mb::umma_desc_sw128(aK + h * (kT * 128) + s * 32), kIdescS, (h | s) != 0);
      mb::tc_commit(&bar_s);
    }
    fetch(j + 1);                                       // its latency hides behind both products and the softmax
    ok = mb::mbar_wait(&bar_s, ph_s, p.status, MB_ST_TIMEOUT_MMA) && ok;
    ph_s ^= 1;
    mb::tc_fence_after();
    // ---- online softmax on this thread's row. The running maximum only moves when the new one is
    // more than 2^8 above it (probabilities then stay below 256, exact enough in bf16 / fp32), so the
    // O accumulator in TMEM is rescaled on few tiles.
    {
      float sv[kT];
#pragma unroll
      for (int c = 0; c < kT / 16; ++c) mb::tmem_ld16(t_row + c * 16, sv + c * 16);
      float mx = -INFINITY;
      const int tok0 = j * kT;
      if (tok0 + kT <= first_limit) {                    // the whole tile is visible to every row of this CTA
#pragma unroll
        for (int i = 0; i < kT; ++i) {
          sv[i] *= sc_log2;
          mx = fmaxf(mx, sv[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < kT; ++i) {
          const float v = (tok0 + i < limit) ? sv[i] * sc_log2 : -INFINITY;
          sv[i] = v;
          mx = fmaxf(mx, v);
        }
      }
      float alpha = 1.f;
      const bool move = mx > m_run + 8.f;                // also true on a row's first finite tile
      if (move) {
        alpha = ex2(m_run - mx);                         // 0 when the row had seen nothing yet
        m_run = mx;
      }
      if (j > 0 && __any_sync(0xffffffffu, move)) {
#pragma unroll
        for (int c = 0; c < kD / 16; ++c) {
          float ov[16];
          mb::tmem_ld16(t_row + 64 + c * 16, ov);
#pragma unroll
          for (int i = 0; i < 16; ++i) ov[i] *= alpha;
          mb::tmem_st16(t_row + 64 + c * 16, ov);
        }
        mb::tmem_st_wait();
      }
      const float m_use = m_run == -INFINITY ? 0.f : m_run;
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 pk;
        uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = ex2(sv[c * 8 + 2 * i] - m_use), b = ex2(sv[c * 8 + 2 * i + 1] - m_use);
          const __nv_bfloat162 pb = __floats2bfloat162_rn(a, b);
          rs += a + b;
          pw[i] = *reinterpret_cast<const uint32_t*>(&pb);
        }
        *reinterpret_cast<uint4*>(sP + sw_off(tid, c)) = pk;
      }
      l_run = l_run * alpha + rs;
    }
    fence_async_smem();
    mb::tc_fence_before();
    // a wait that ran out in any thread (the status word says so) ends the loop for the whole CTA
    ok = __syncthreads_and(ok) != 0;
    if (!ok) break;
    // ---- O += P V (accumulated in TMEM across tiles)
    if (tid == 0) {
      mb::tc_fence_after();
#pragma unroll
      for (int s = 0; s < 4; ++s)
        mb::umma_f16(tmem + 64, mb::umma_desc_sw128(aP + s * 32),
                     VMN ? mb::umma_desc_sw128_mn(aV + s * 2048, kT * 128, 1024)   // 16 tokens = two 8-row groups on
                         : mb::umma_desc_sw128(aV + s * 32),
                     kIdescO, (j | s) != 0);
      mb::tc_commit(&bar_o);
    }
  }
  if (ok && tiles > 0) {
    ok = mb::mbar_wait(&bar_o, ph_o, p.status, MB_ST_TIMEOUT_MMA) && ok;
    mb::tc_fence_after();
  }
  if (ok) {                                               // uniform: tcgen05.ld is a whole-warp instruction
    const float vmul = FP8 ? (*p.v_scale) * 256.f : 1.f;
    const float inv = l_run > 0.f ? vmul / l_run : 0.f;
    uint4* dst = reinterpret_cast<uint4*>(p.out + ((size_t)(qs + (row_ok ? qi : 0)) * p.Hq + head) * kD);
#pragma unroll
    for (int c = 0; c < kD / 16; ++c) {
      float ov[16];
      mb::tmem_ld16(t_row + 64 + c * 16, ov);             // every lane reads; only rows of the sequence store
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        uint4 w;
        __nv_bfloat162* wb = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
        for (int i = 0; i < 4; ++i) wb[i] = __floats2bfloat162_rn(ov[h2 * 8 + 2 * i] * inv, ov[h2 * 8 + 2 * i + 1] * inv);
        if (row_ok) dst[c * 2 + h2] = w;
      }
    }
  }
  mb::tc_fence_before();
  __syncthreads();
  if (warp == 0) mb::tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

struct MbAttnTcArgs {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const int* block_table;
  const int* q_start;
  const int* q_len;
  const int* ctx_len;
  const float* k_scale;
  const float* v_scale;
  void* out;
  uint32_t* status;
  long long num_blocks;
  int max_blocks, num_seqs, max_q_len, Hq, Hkv, D, block_size, cache_fp8;
  float scale;
  int v_mn;      // 1: V staged as stored and read as an MN-major operand (no transposition)
};

// Causal paged attention for prefill chunks (head dim 128). Returns 0, MB_ERR_* or a CUDA error.
extern "C" int mb_attn_prefill_tc(const MbAttnTcArgs* a, cudaStream_t stream) {
  if (!a || !a->q || !a->k_cache || !a->v_cache || !a->block_table || !a->out) return MB_ERR_BAD_ARG;
  if ((a->D != 128 && a->D != 256) || a->num_seqs <= 0 || a->Hkv <= 0 || a->Hq % a->Hkv || a->max_q_len <= 0) return MB_ERR_UNSUPPORTED;
  if (a->cache_fp8 && (!a->k_scale || !a->v_scale)) return MB_ERR_BAD_ARG;
  TcParams p;
  p.q = (const __nv_bfloat16*)a->q; p.k_cache = a->k_cache; p.v_cache = a->v_cache;
  p.block_table = a->block_table; p.max_blocks = a->max_blocks;
  p.q_start = a->q_start; p.q_len = a->q_len; p.ctx_len = a->ctx_len;
  p.Hq = a->Hq; p.Hkv = a->Hkv; p.block_size = a->block_size; p.num_blocks = a->num_blocks;
  p.scale = a->scale; p.k_scale = a->k_scale; p.v_scale = a->v_scale;
  p.out = (__nv_bfloat16*)a->out; p.status = a->status;
  const size_t smem = (size_t)(a->D / 64) * (kQ + 2 * kT) * 128 + kQ * 128 + 1024;
  static bool configured = false;
  if (!configured) {
    const int s128 = 2 * (kQ + 2 * kT) * 128 + kQ * 128 + 1024, s256 = 4 * (kQ + 2 * kT) * 128 + kQ * 128 + 1024;
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<128, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, s128);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_prefill_tc_kernel<128, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, s128);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_prefill_tc_kernel<128, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, s128);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_prefill_tc_kernel<128, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, s128);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_prefill_tc_kernel<256, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, s256);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_prefill_tc_kernel<256, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, s256);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const dim3 grid((a->max_q_len + kQ - 1) / kQ, a->Hq, a->num_seqs);
  if (a->D == 256) {
    if (a->cache_fp8) return (int)mb::launch_kernel(attn_prefill_tc_kernel<256, true, true>, grid, dim3(128), smem, stream, p);
    return (int)mb::launch_kernel(attn_prefill_tc_kernel<256, false, true>, grid, dim3(128), smem, stream, p);
  }
  if (a->v_mn) {
    if (a->cache_fp8) return (int)mb::launch_kernel(attn_prefill_tc_kernel<128, true, true>, grid, dim3(128), smem, stream, p);
    return (int)mb::launch_kernel(attn_prefill_tc_kernel<128, false, true>, grid, dim3(128), smem, stream, p);
  }
  if (a->cache_fp8) return (int)mb::launch_kernel(attn_prefill_tc_kernel<128, true, false>, grid, dim3(128), smem, stream, p);
  return (int)mb::launch_kernel(attn_prefill_tc_kernel<128, false, false>, grid, dim3(128), smem, stream, p);
}
