// Tensor-parallel collectives fused with the op that consumes them, over NVLink peer
// memory (sm_100a, NVSwitch).
//
//   mb_tp_reduce_norm   all-reduce of a row-parallel projection's bf16 partial sums
//                       + residual add + RMSNorm + activation quantiser (bf16 / fp8 per row /
//                       fp8 per 128 channels / NVFP4), in one kernel. Two protocols:
//                         one-shot  every rank reduces every row itself (one switch-side
//                                   reduction per 16 bytes through `multimem.ld_reduce`, or
//                                   one 16-byte load per peer when the group has no multicast
//                                   mapping) and writes the quantised rows locally: one
//                                   barrier per call, for decode-sized batches;
//                         two-shot  rank r reduces rows [r*ceil(M/size), ...) only and
//                                   broadcasts the *quantised* rows (4.5 bits per value for
//                                   NVFP4 instead of 16) with `multimem.st` into every rank's
//                                   activation buffer, so the GEMM that follows reads the
//                                   gathered operand from local memory (all-gather fused into
//                                   the producer of the operand): two barriers per call.
//                         packets   for the smallest batches there is no barrier at all: every rank
//                                   broadcasts its partial rows as 8-byte packets (two bf16 values
//                                   + a 4-byte tag that changes every call) with `multimem.st`, and
//                                   every rank polls its own landing zone until all `size` packets
//                                   of a position carry the current tag, then sums them in rank
//                                   order. One NVLink hop per call instead of a signal hop plus a
//                                   load round trip; twice the bytes, so only below ~1.5 MB.
//   mb_tp_argmax_merge  vocab-parallel greedy selection: every rank publishes one
//                       (max logit, global index) pair per row; all ranks pull the pairs of
//                       their peers and keep the best (8 bytes per rank per row instead of an
//                       all-gather of the logits).
//   mb_tp_barrier       the barrier alone (used to close a forward pass whose last reduction
//                       was one-shot, so that buffer reuse by the next pass is ordered).
//
// Barrier protocol. Counters live in symmetric memory (same offset on every rank). Every
// call adds 1 to the `arrive` counter of every rank (one `multimem.red` through the switch,
// or one `red.release.sys` per peer) once the kernel in front of it has completed, and waits
// until its own counter reaches (epoch + 1) * size, where `epoch` is a device-resident call
// count (so a captured CUDA graph replays correctly). The last CTA of a call advances the
// epoch. Two-shot calls repeat this on a `done` counter after their broadcast stores have
// been fenced. Every wait is bounded by a cycle budget given at run time; on expiry the
// kernel records MB_ST_TIMEOUT_PEER in the status word, skips its data phase and returns.
//
// No TMA load touches peer memory and no load is a cluster multicast; peers are reached
// with plain loads / stores, `multimem.ld_reduce`, `multimem.st` and `multimem.red` only.
//
// The reference all-reduces with NCCL after the local GEMM and runs the norm as a separate
// kernel (crates/model-layers/src/layers/qwen3_attention/trait_impl/decode_inner.rs:109-117,
// crates/model-engine/src/model/impl_a3_lm_head.rs:157-201).
#include "common.cuh"

namespace {

enum { OUT_BF16 = 0, OUT_FP8_ROW = 1, OUT_FP8_G128 = 2, OUT_NVFP4 = 3, OUT_NONE = 4 };

struct TpSync {
  uint32_t* arrive;            // this rank's arrival counter
  uint32_t* arrive_mc;         // multicast alias of all ranks' arrival counters, or null
  uint32_t* arrive_peer[8];    // every rank's arrival counter (no-multicast path)
  uint32_t* done;              // same three for the completion counter (two-shot)
  uint32_t* done_mc;
  uint32_t* done_peer[8];
  uint32_t* epoch;             // local: [0] calls completed on this barrier, [1] two-shot calls, [2] packet-protocol calls
  uint32_t* cta_done;          // local: CTAs of the running call that have finished
  uint32_t* status;
  long long wait_cycles;
  int size, rank;
};

struct TpNormParams {
  TpSync s;
  int M, K;
  int row_lo, row_hi;          // rows this rank reduces
  int out_mode;
  const __nv_bfloat16* partial_mc;      // multicast alias of the partial buffers, or null
  const __nv_bfloat16* partial[8];      // every rank's partial buffer [M, K]
  const __nv_bfloat16* residual;        // local [M, K] or null
  __nv_bfloat16* residual_out;          // local [M, K] or null
  __nv_bfloat16* residual_out_mc;       // multicast alias (two-shot, gathered residual) or null
  const __nv_bfloat16* w;
  int do_norm, w_plus_one;
  float eps;
  uint8_t* out;                // quantised rows (multicast alias when two-shot)
  long long out_ld;            // bytes for fp8 / fp4, elements for bf16
  __nv_bfloat16* out_bf16;     // extra bf16 copy of the normalised rows, or null
  long long out_bf16_ld;
  float* scale;
  int scale_ld;
  uint8_t* sf;
  int sf_k64;
  float static_gs;
  // packet protocol: landing zones [2 parity][size][ll_rows][K / 2] of 8-byte packets
  uint2* ll;                   // this rank's zones
  uint2* ll_mc;                // multicast alias, or null
  uint2* ll_peer[8];           // every rank's zones (no-multicast path)
  int ll_rows;
  const __nv_bfloat16* partial_local;   // this rank's partial [M, K]
};

__device__ __forceinline__ void multimem_red_add_release(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_st_f32(void* mc, uint32_t bits) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc), "f"(__uint_as_float(bits)) : "memory");
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_relaxed_sys_v2(const void* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

// one signal to the counter of every rank (the caller's own included)
__device__ __forceinline__ void signal_all(uint32_t* mc, uint32_t* const* peer, int size) {
  __threadfence_system();
  if (mc) {
    multimem_red_add_release(mc, 1u);
  } else {
    for (int r = 0; r < size; ++r) mb::red_add_release_sys(peer[r], 1u);
  }
}
// bounded spin until the counter has reached `want` (wrap-safe)
__device__ __forceinline__ bool wait_count(const uint32_t* p, uint32_t want, uint32_t* status, long long budget) {
  const long long t0 = clock64();
  while ((int)(mb::ld_acquire_sys(p) - want) < 0) {
    if (clock64() - t0 > budget) {
      if (status) atomicCAS(status, 0u, MB_ST_TIMEOUT_PEER);
      return false;
    }
  }
  return true;
}

// Entry half of a call: CTA 0 announces this rank, every CTA waits for all ranks. Returns the
// epoch through `e` and false when the wait ran out.
__device__ __forceinline__ bool sync_enter(const TpSync& s, uint32_t* sh, uint2& e) {
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) signal_all(s.arrive_mc, s.arrive_peer, s.size);
    const uint32_t ep = *reinterpret_cast<volatile uint32_t*>(s.epoch);
    sh[0] = ep;
    sh[2] = *reinterpret_cast<volatile uint32_t*>(s.epoch + 1);
    sh[1] = wait_count(s.arrive, (ep + 1u) * (uint32_t)s.size, s.status, s.wait_cycles) ? 1u : 0u;
  }
  __syncthreads();
  e = make_uint2(sh[0], sh[2]);
  return sh[1] != 0u;
}
// Exit half: the last CTA advances the epoch (and, for two-shot calls, announces that this
// rank's broadcast stores are complete); with `wait_done` every CTA then waits for all ranks.
__device__ __forceinline__ void sync_exit(const TpSync& s, uint2 e, bool two_shot, bool ok) {
  __syncthreads();
  if (threadIdx.x == 0) {
    // one fence per CTA, after the CTA barrier, orders every thread's broadcast stores before the
    // completion count (and, through the last CTA's release, before the peers' acquire)
    if (two_shot) __threadfence_system();
    const uint32_t prev = atomicAdd(s.cta_done, 1u);
    if (prev == gridDim.x - 1) {
      if (two_shot) {
        signal_all(s.done_mc, s.done_peer, s.size);
        *reinterpret_cast<volatile uint32_t*>(s.epoch + 1) = e.y + 1u;
      }
      *reinterpret_cast<volatile uint32_t*>(s.cta_done) = 0u;
      *reinterpret_cast<volatile uint32_t*>(s.epoch) = e.x + 1u;
    }
    if (two_shot && ok) wait_count(s.done, (e.y + 1u) * (uint32_t)s.size, s.status, s.wait_cycles);
  }
}

template <bool MC>
__device__ __forceinline__ void st16(void* p, const uint4& v) {
  if (MC) mb::multimem_st_v4(p, v);
  else *reinterpret_cast<uint4*>(p) = v;
}
template <bool MC>
__device__ __forceinline__ void st4(void* p, uint32_t v) {
  if (MC) multimem_st_f32(p, v);
  else *reinterpret_cast<uint32_t*>(p) = v;
}

__device__ __forceinline__ void unpack16(const uint4& v0, const uint4& v1, float* x) {
  const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&v0);
  const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&v1);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(h0[i]), c = __bfloat1622float2(h1[i]);
    x[2 * i] = a.x; x[2 * i + 1] = a.y; x[8 + 2 * i] = c.x; x[8 + 2 * i + 1] = c.y;
  }
}
__device__ __forceinline__ void pack16(const float* y, uint4& o0, uint4& o1) {
  __nv_bfloat162* q0 = reinterpret_cast<__nv_bfloat162*>(&o0);
  __nv_bfloat162* q1 = reinterpret_cast<__nv_bfloat162*>(&o1);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    q0[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
    q1[i] = __floats2bfloat162_rn(y[8 + 2 * i], y[8 + 2 * i + 1]);
  }
}

__device__ __forceinline__ void multimem_st_v2(void* mc, uint32_t a, uint32_t b) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc), "f"(__uint_as_float(a)),
               "f"(__uint_as_float(b))
               : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_v2(void* p, uint32_t a, uint32_t b) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

// Packet protocol, one row: broadcast this rank's 16 values per thread as 8 packets, then poll
// the local landing zones of all ranks until every packet carries `tag`; x = bf16(sum in rank
// order). Returns false when the bounded wait ran out.
__device__ __forceinline__ bool ll_exchange_row(const TpNormParams& p, int m, int tid, uint32_t tag,
                                                uint32_t parity, float* x) {
  const int K = p.K, size = p.s.size;
  const size_t row_pk = (size_t)(K >> 1);                              // packets per row
  const size_t zone = (size_t)p.ll_rows * row_pk;                      // packets per (parity, rank)
  const size_t mine = ((size_t)parity * size + p.s.rank) * zone + (size_t)m * row_pk + (size_t)tid * 8;
  const uint4 v0 = *reinterpret_cast<const uint4*>(p.partial_local + (size_t)m * K + tid * 16);
  const uint4 v1 = *reinterpret_cast<const uint4*>(p.partial_local + (size_t)m * K + tid * 16 + 8);
  const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  if (p.ll_mc) {
#pragma unroll
    for (int j = 0; j < 8; ++j) multimem_st_v2(p.ll_mc + mine + j, w[j], tag);
  } else {
    for (int r = 0; r < size; ++r) {
#pragma unroll
      for (int j = 0; j < 8; ++j) st_relaxed_sys_v2(p.ll_peer[r] + mine + j, w[j], tag);
    }
  }
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.f;
  const long long t0 = clock64();
  for (int r = 0; r < size; ++r) {
    const uint2* src = p.ll + ((size_t)parity * size + r) * zone + (size_t)m * row_pk + (size_t)tid * 8;
    uint4 q[4];
    bool ready;
    do {
#pragma unroll
      for (int j = 0; j < 4; ++j) q[j] = ld_relaxed_sys_v4(src + 2 * j);
      ready = true;
#pragma unroll
      for (int j = 0; j < 4; ++j) ready = ready && q[j].y == tag && q[j].w == tag;
      if (!ready && clock64() - t0 > p.s.wait_cycles) {
        if (p.s.status) atomicCAS(p.s.status, 0u, MB_ST_TIMEOUT_PEER);
        return false;
      }
    } while (!ready);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q[j].x));
      const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q[j].z));
      acc[4 * j] += a.x; acc[4 * j + 1] += a.y; acc[4 * j + 2] += c.x; acc[4 * j + 3] += c.y;
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) x[i] = __bfloat162float(__float2bfloat16(acc[i]));
  return true;
}

// One CTA per row at a time; thread t owns the 16 channels [16 t, 16 t + 16). K % 64 == 0,
// K <= 8192. PROTO: 0 one-shot behind a barrier, 1 two-shot (outputs are multicast aliases),
// 2 packets (no barrier; epoch word [2] counts these calls and gives the tag and the parity).
template <int PROTO>
__global__ void __launch_bounds__(512) tp_reduce_norm_kernel(const TpNormParams p) {
  constexpr bool TWO = PROTO == 1;
  __shared__ float red[64];
  __shared__ uint32_t sh[3];
  const int tid = threadIdx.x, nt = blockDim.x;
  const int K = p.K, nblk = K >> 4;
  const bool active = tid < nblk;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  uint2 e = make_uint2(0u, 0u);
  bool ok = true;
  uint32_t ll_epoch = 0;
  if (PROTO == 2) {
    ll_epoch = *reinterpret_cast<volatile uint32_t*>(p.s.epoch + 2);
  } else {
    ok = sync_enter(p.s, sh, e);
  }
  if (ok) {
    for (int m = p.row_lo + blockIdx.x; m < p.row_hi; m += gridDim.x) {
      float x[16];
      float ss = 0.f, mx = 0.f;
      if (PROTO == 2) {
        // every thread takes part (a thread beyond the row has no packets and no work)
        bool got = true;
        if (active) got = ll_exchange_row(p, m, tid, ll_epoch + 1u, ll_epoch & 1u, x);
        if (__syncthreads_count(got ? 0 : 1) > 0) { ok = false; break; }
      }
      if (active) {
        const size_t off = (size_t)m * K + (size_t)tid * 16;
        if (PROTO == 2) {
          // x already holds the sum
        } else if (p.partial_mc) {
          const uint4 v0 = mb::multimem_ld_reduce_bf16x8(p.partial_mc + off);
          const uint4 v1 = mb::multimem_ld_reduce_bf16x8(p.partial_mc + off + 8);
          unpack16(v0, v1, x);
        } else {
          float acc[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = 0.f;
          for (int r = 0; r < p.s.size; ++r) {
            const uint4 v0 = ld_relaxed_sys_v4(p.partial[r] + off);
            const uint4 v1 = ld_relaxed_sys_v4(p.partial[r] + off + 8);
            float t[16];
            unpack16(v0, v1, t);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] += t[i];
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) x[i] = __bfloat162float(__float2bfloat16(acc[i]));
        }
        if (p.residual) {
          const uint4 r0 = *reinterpret_cast<const uint4*>(p.residual + off);
          const uint4 r1 = *reinterpret_cast<const uint4*>(p.residual + off + 8);
          float t[16];
          unpack16(r0, r1, t);
#pragma unroll
          for (int i = 0; i < 16; ++i) x[i] = __bfloat162float(__float2bfloat16(x[i] + t[i]));
        }
        if (p.residual_out || p.residual_out_mc) {
          uint4 o0, o1;
          pack16(x, o0, o1);
          if (p.residual_out) {
            *reinterpret_cast<uint4*>(p.residual_out + off) = o0;
            *reinterpret_cast<uint4*>(p.residual_out + off + 8) = o1;
          }
          if (TWO && p.residual_out_mc) {
            mb::multimem_st_v4(p.residual_out_mc + off, o0);
            mb::multimem_st_v4(p.residual_out_mc + off + 8, o1);
          }
        }
        if (p.do_norm) {
          float w[16];
          if (p.w) {
            const uint4 w0 = __ldg(reinterpret_cast<const uint4*>(p.w + tid * 16));
            const uint4 w1 = __ldg(reinterpret_cast<const uint4*>(p.w + tid * 16) + 1);
            unpack16(w0, w1, w);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) w[i] = 1.f;
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            ss += x[i] * x[i];
            x[i] *= p.w_plus_one ? (w[i] + 1.f) : w[i];
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) mx = fmaxf(mx, fabsf(x[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = 0.f;
      }
      if (p.out_mode == OUT_NONE && !p.out_bf16) continue;      // uniform across the CTA
      float inv = 1.f, amax = mx;
      if (p.do_norm || p.out_mode == OUT_FP8_ROW || p.out_mode == OUT_NVFP4) {
        ss = mb::warp_sum(ss);
        mx = mb::warp_max(mx);
        const int w = tid >> 5, l = tid & 31, nw = (nt + 31) >> 5;
        __syncthreads();                                       // red[] of the previous row is consumed
        if (l == 0) { red[w] = ss; red[32 + w] = mx; }
        __syncthreads();
        float a = l < nw ? red[l] : 0.f, c = l < nw ? red[32 + l] : 0.f;
        a = mb::warp_sum(a);
        c = mb::warp_max(c);
        if (p.do_norm) inv = rsqrtf(a / (float)K + p.eps);
        amax = c * inv;
      }
      float y[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) y[i] = x[i] * inv;
      if (active && (p.out_bf16 || p.out_mode == OUT_BF16)) {
        uint4 o0, o1;
        pack16(y, o0, o1);
        if (p.out_bf16) {
          __nv_bfloat16* d = p.out_bf16 + (size_t)m * p.out_bf16_ld + tid * 16;
          st16<TWO>(d, o0);
          st16<TWO>(d + 8, o1);
        }
        if (p.out_mode == OUT_BF16) {
          __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.out_ld + tid * 16;
          st16<TWO>(d, o0);
          st16<TWO>(d + 8, o1);
        }
      }
      if (p.out_mode == OUT_FP8_ROW || p.out_mode == OUT_FP8_G128) {
        float sc_inv;
        if (p.out_mode == OUT_FP8_ROW) {
          const float gs = amax > 0.f ? amax / 448.f : 1.f;
          sc_inv = 1.f / gs;
          if (tid == 0) st4<TWO>(p.scale + m, __float_as_uint(gs));
        } else {
          float bm = 0.f;
#pragma unroll
          for (int i = 0; i < 16; ++i) bm = fmaxf(bm, fabsf(y[i]));
          bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
          bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
          bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 4));
          const float sc = bm > 0.f ? bm / 448.f : 1.f;
          sc_inv = 1.f / sc;
          if (active && (tid & 7) == 0) st4<TWO>(p.scale + (size_t)(tid >> 3) * p.scale_ld + m, __float_as_uint(sc));
        }
        uint32_t w4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          w4[i] = (uint32_t)mb::float_to_e4m3(y[4 * i] * sc_inv) | ((uint32_t)mb::float_to_e4m3(y[4 * i + 1] * sc_inv) << 8) |
                  ((uint32_t)mb::float_to_e4m3(y[4 * i + 2] * sc_inv) << 16) | ((uint32_t)mb::float_to_e4m3(y[4 * i + 3] * sc_inv) << 24);
        }
        if (active) st16<TWO>(p.out + (size_t)m * p.out_ld + tid * 16, make_uint4(w4[0], w4[1], w4[2], w4[3]));
      } else if (p.out_mode == OUT_NVFP4) {
        const float gs = p.static_gs > 0.f ? p.static_gs : (amax > 0.f ? amax / (6.f * 448.f) : 1.f);
        if (tid == 0) st4<TWO>(p.scale + m, __float_as_uint(gs));
        float bmax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(y[i]));
        const uint32_t sfc = mb::float_to_e4m3(bmax / (6.f * gs));
        const float sff = mb::e4m3_to_float((uint8_t)sfc);
        const float qi = sff > 0.f ? 1.f / (sff * gs) : 0.f;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) lo |= mb::e2m1x2_pack(y[2 * i] * qi, y[2 * i + 1] * qi) << (8 * i);
#pragma unroll
        for (int i = 0; i < 4; ++i) hi |= mb::e2m1x2_pack(y[8 + 2 * i] * qi, y[8 + 2 * i + 1] * qi) << (8 * i);
        // 16-byte stores: the even lane of a pair writes both lanes' 8 bytes; the first lane of
        // a group of four writes the group's four scale factors (one 64-channel group)
        const uint32_t lo2 = __shfl_down_sync(0xffffffffu, lo, 1), hi2 = __shfl_down_sync(0xffffffffu, hi, 1);
        uint32_t sf4 = sfc;
        sf4 |= __shfl_down_sync(0xffffffffu, sfc, 1) << 8;
        sf4 |= __shfl_down_sync(0xffffffffu, sfc, 2) << 16;
        sf4 |= __shfl_down_sync(0xffffffffu, sfc, 3) << 24;
        if (active && (tid & 1) == 0)
          st16<TWO>(p.out + (size_t)m * p.out_ld + tid * 8, make_uint4(lo, hi, lo2, hi2));
        if (active && (tid & 3) == 0) {
          uint8_t* sf_blk = p.sf + (size_t)(m >> 7) * p.sf_k64 * 512;
          st4<TWO>(sf_blk + (size_t)(tid >> 2) * 512 + mb::sf_tile_offset(m & 127, 0), sf4);
        }
      }
    }
  }
  if (PROTO == 2) {
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t prev = atomicAdd(p.s.cta_done, 1u);
      if (prev == gridDim.x - 1) {
        *reinterpret_cast<volatile uint32_t*>(p.s.cta_done) = 0u;
        *reinterpret_cast<volatile uint32_t*>(p.s.epoch + 2) = ll_epoch + 1u;
      }
    }
  } else {
    sync_exit(p.s, e, TWO, ok);
  }
}

// Greedy selection over a vocabulary sharded across ranks: `pairs[r]` is rank r's array of
// (max logit bits, global index) per row. One CTA; thread m merges row m. First maximum wins
// (a lower global index wins ties, as in the single-rank argmax).
struct TpMergeParams {
  TpSync s;
  int M;
  const uint2* pairs[8];
  int* out_ids;
  int* feed;
};
__global__ void __launch_bounds__(1024) tp_argmax_merge_kernel(const TpMergeParams p) {
  __shared__ uint32_t sh[3];
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  uint2 e;
  const bool ok = sync_enter(p.s, sh, e);
  if (ok) {
    for (int m = threadIdx.x; m < p.M; m += blockDim.x) {
      float best = -INFINITY;
      int bidx = 0x7fffffff;
      for (int r = 0; r < p.s.size; ++r) {
        const uint2 v = ld_relaxed_sys_v2(p.pairs[r] + m);
        const float f = __uint_as_float(v.x);
        const int i = (int)v.y;
        if (f > best || (f == best && i < bidx)) { best = f; bidx = i; }
      }
      if (bidx == 0x7fffffff) bidx = 0;
      p.out_ids[m] = bidx;
      if (p.feed) p.feed[m] = bidx;
    }
  }
  sync_exit(p.s, e, false, ok);
}

__global__ void tp_barrier_kernel(const TpSync s) {
  __shared__ uint32_t sh[3];
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  uint2 e;
  const bool ok = sync_enter(s, sh, e);
  sync_exit(s, e, false, ok);
}

}  // namespace

extern "C" {

struct MbTpSync {
  void* arrive; void* arrive_mc; void* arrive_peer[8];
  void* done; void* done_mc; void* done_peer[8];
  void* epoch; void* cta_done; void* status;
  long long wait_cycles;
  int size, rank;
};

struct MbTpNormArgs {
  MbTpSync sync;
  int M, K, two_shot, out_mode;
  const void* partial_mc;
  const void* partial[8];
  const void* residual;
  void* residual_out;
  void* residual_out_mc;
  const void* w;
  int do_norm, w_plus_one;
  float eps;
  void* out;
  long long out_ld;
  void* out_bf16;
  long long out_bf16_ld;
  void* scale;
  int scale_ld;
  void* sf;
  int sf_k64;
  float static_gs;
  int max_ctas;
  // packet protocol (two_shot == 2)
  void* ll;
  void* ll_mc;
  void* ll_peer[8];
  int ll_rows;
};

static int fill_sync(const MbTpSync& a, TpSync& s) {
  if (!a.arrive || !a.epoch || !a.cta_done || a.size < 1 || a.size > 8 || a.rank < 0 || a.rank >= a.size)
    return MB_ERR_BAD_ARG;
  s.arrive = reinterpret_cast<uint32_t*>(a.arrive);
  s.arrive_mc = reinterpret_cast<uint32_t*>(a.arrive_mc);
  s.done = reinterpret_cast<uint32_t*>(a.done);
  s.done_mc = reinterpret_cast<uint32_t*>(a.done_mc);
  for (int r = 0; r < 8; ++r) {
    s.arrive_peer[r] = reinterpret_cast<uint32_t*>(a.arrive_peer[r]);
    s.done_peer[r] = reinterpret_cast<uint32_t*>(a.done_peer[r]);
    if (r < a.size && !a.arrive_mc && !a.arrive_peer[r]) return MB_ERR_BAD_ARG;
  }
  s.epoch = reinterpret_cast<uint32_t*>(a.epoch);
  s.cta_done = reinterpret_cast<uint32_t*>(a.cta_done);
  s.status = reinterpret_cast<uint32_t*>(a.status);
  s.wait_cycles = a.wait_cycles > 0 ? a.wait_cycles : MB_WAIT_CYCLES;
  s.size = a.size;
  s.rank = a.rank;
  return MB_OK;
}

int mb_tp_reduce_norm(const MbTpNormArgs* a, cudaStream_t stream) {
  if (!a || a->M <= 0 || a->K <= 0) return MB_ERR_BAD_ARG;
  if (a->K % 64 || a->K > 8192) return MB_ERR_UNSUPPORTED;
  TpNormParams p{};
  int rc = fill_sync(a->sync, p.s);
  if (rc) return rc;
  const int size = p.s.size;
  if (a->two_shot == 1 && (!a->sync.done || (!a->sync.done_mc && !a->sync.done_peer[0]))) return MB_ERR_BAD_ARG;
  if (a->two_shot == 2) {
    if (!a->ll || a->ll_rows < a->M || !a->partial[p.s.rank]) return MB_ERR_BAD_ARG;
    if (!a->ll_mc)
      for (int r = 0; r < size; ++r)
        if (!a->ll_peer[r]) return MB_ERR_BAD_ARG;
  } else if (!a->partial_mc) {
    for (int r = 0; r < size; ++r)
      if (!a->partial[r]) return MB_ERR_BAD_ARG;
  }
  if (a->out_mode < OUT_BF16 || a->out_mode > OUT_NONE) return MB_ERR_BAD_ARG;
  if (a->out_mode != OUT_NONE && !a->out) return MB_ERR_BAD_ARG;
  if (a->out_mode == OUT_NVFP4 && (!a->sf || !a->scale || a->sf_k64 * 64 < a->K)) return MB_ERR_BAD_ARG;
  if ((a->out_mode == OUT_FP8_ROW || a->out_mode == OUT_FP8_G128) && !a->scale) return MB_ERR_BAD_ARG;
  if (a->out_mode == OUT_FP8_G128 && a->K % 128) return MB_ERR_UNSUPPORTED;
  p.M = a->M; p.K = a->K; p.out_mode = a->out_mode;
  if (a->two_shot == 1) {
    const int per = (a->M + size - 1) / size;
    p.row_lo = per * p.s.rank < a->M ? per * p.s.rank : a->M;
    p.row_hi = p.row_lo + per < a->M ? p.row_lo + per : a->M;
  } else {
    p.row_lo = 0; p.row_hi = a->M;
  }
  p.partial_mc = reinterpret_cast<const __nv_bfloat16*>(a->partial_mc);
  for (int r = 0; r < 8; ++r) p.partial[r] = reinterpret_cast<const __nv_bfloat16*>(a->partial[r]);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a->residual);
  p.residual_out = reinterpret_cast<__nv_bfloat16*>(a->residual_out);
  p.residual_out_mc = reinterpret_cast<__nv_bfloat16*>(a->residual_out_mc);
  p.w = reinterpret_cast<const __nv_bfloat16*>(a->w);
  p.do_norm = a->do_norm; p.w_plus_one = a->w_plus_one; p.eps = a->eps;
  p.out = reinterpret_cast<uint8_t*>(a->out); p.out_ld = a->out_ld;
  p.out_bf16 = reinterpret_cast<__nv_bfloat16*>(a->out_bf16); p.out_bf16_ld = a->out_bf16_ld;
  p.scale = reinterpret_cast<float*>(a->scale); p.scale_ld = a->scale_ld;
  p.sf = reinterpret_cast<uint8_t*>(a->sf); p.sf_k64 = a->sf_k64;
  p.static_gs = a->static_gs;
  p.ll = reinterpret_cast<uint2*>(a->ll);
  p.ll_mc = reinterpret_cast<uint2*>(a->ll_mc);
  for (int r = 0; r < 8; ++r) p.ll_peer[r] = reinterpret_cast<uint2*>(a->ll_peer[r]);
  p.ll_rows = a->ll_rows;
  p.partial_local = p.partial[p.s.rank];
  const int rows = p.row_hi - p.row_lo;
  const int cap = a->max_ctas > 0 ? a->max_ctas : 128;        // every CTA must be resident: they wait on one another
  const int grid = rows < 1 ? 1 : (rows < cap ? rows : cap);
  const int threads = ((a->K / 16) + 31) / 32 * 32;
  const bool pdl = mb_pdl_enabled() >= 1;
  if (a->two_shot == 2)
    return (int)mb::launch_kernel_ex(tp_reduce_norm_kernel<2>, dim3(grid), dim3(threads), 0, stream, 1, pdl, p);
  if (a->two_shot == 1)
    return (int)mb::launch_kernel_ex(tp_reduce_norm_kernel<1>, dim3(grid), dim3(threads), 0, stream, 1, pdl, p);
  return (int)mb::launch_kernel_ex(tp_reduce_norm_kernel<0>, dim3(grid), dim3(threads), 0, stream, 1, pdl, p);
}

struct MbTpMergeArgs {
  MbTpSync sync;
  int M;
  const void* pairs[8];
  int* out_ids;
  int* feed;
};

int mb_tp_argmax_merge(const MbTpMergeArgs* a, cudaStream_t stream) {
  if (!a || a->M <= 0 || !a->out_ids) return MB_ERR_BAD_ARG;
  TpMergeParams p{};
  int rc = fill_sync(a->sync, p.s);
  if (rc) return rc;
  for (int r = 0; r < 8; ++r) {
    p.pairs[r] = reinterpret_cast<const uint2*>(a->pairs[r]);
    if (r < p.s.size && !a->pairs[r]) return MB_ERR_BAD_ARG;
  }
  p.M = a->M; p.out_ids = a->out_ids; p.feed = a->feed;
  int threads = (a->M + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  return (int)mb::launch_kernel_ex(tp_argmax_merge_kernel, dim3(1), dim3(threads), 0, stream, 1,
                                   mb_pdl_enabled() >= 1, p);
}

int mb_tp_barrier(const MbTpSync* a, cudaStream_t stream) {
  if (!a) return MB_ERR_BAD_ARG;
  TpSync s{};
  int rc = fill_sync(*a, s);
  if (rc) return rc;
  return (int)mb::launch_kernel_ex(tp_barrier_kernel, dim3(1), dim3(32), 0, stream, 1, mb_pdl_enabled() >= 1, s);
}

}  // extern "C"
