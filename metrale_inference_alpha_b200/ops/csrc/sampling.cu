// Token selection on the device (the reference samples on the host and only runs
// argmax on the GPU; here the whole pipeline stays on the device so a decode step
// needs a 4-byte-per-row readback and nothing else).
//
//   mb_argmax        row argmax over bf16 or fp32 logits, first maximum wins, optional
//                    two-id mask, optional top-1 log-probability (online softmax), and an
//                    optional "feed" cell so the next step can read its input token from
//                    device memory without a host round trip.
//   mb_sample        per-row temperature -> top-k -> min-p -> top-p -> multinomial with a
//                    counter-based RNG keyed by (seed, step). Thresholds are found by
//                    bisection over the order-preserving integer image of the logits, so
//                    no sort and no workspace beyond the fp32 row are needed.
//   mb_apply_penalties  repetition / presence / frequency penalties and logit bias from a
//                    per-row list of (token, count, in_prompt) triples.
//
// Reference behaviour covered: kernels/gb10/common/argmax_bf16.cu, argmax_feed.cu and the
// host sampler crates/sampling/src/{sample_impl.rs,penalties.rs,feed_argmax.rs}.
#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t ordered_u32(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float from_ordered(uint32_t o) {
  const uint32_t u = (o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o;
  return __uint_as_float(u);
}

template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, size_t i);
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
  return __bfloat162float(p[i]);
}

template <typename T>
__global__ void __launch_bounds__(1024)
argmax_kernel(const T* __restrict__ logits, long long ld, int V, int* __restrict__ out_ids,
              float* __restrict__ out_logprob, int mask_a, int mask_b, int* __restrict__ feed,
              const int* __restrict__ row_map, uint2* __restrict__ pair_out, int idx_offset) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ float s_red[32];
  const int row = blockIdx.x;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const T* x = logits + (size_t)row * ld;
  float best = -INFINITY;
  int bidx = 0x7fffffff;
  if (sizeof(T) == 4 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    // 16-byte loads: four logits per thread per step (ascending index order inside a thread keeps
    // the first-maximum rule)
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const int V4 = V >> 2;
    for (int i4 = threadIdx.x; i4 < V4; i4 += blockDim.x) {
      const float4 q = x4[i4];
      const float vv[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = i4 * 4 + k;
        if (i == mask_a || i == mask_b) continue;
        if (vv[k] > best || (vv[k] == best && i < bidx)) { best = vv[k]; bidx = i; }
      }
    }
    for (int i = (V4 << 2) + threadIdx.x; i < V; i += blockDim.x) {
      if (i == mask_a || i == mask_b) continue;
      const float v = ld_logit<T>(x, i);
      if (v > best || (v == best && i < bidx)) { best = v; bidx = i; }
    }
  } else if (sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    // bf16 logits: eight per 16-byte load (the decode step's lm_head writes bf16)
    const uint4* x8 = reinterpret_cast<const uint4*>(x);
    const int V8 = V >> 3;
    for (int i8 = threadIdx.x; i8 < V8; i8 += blockDim.x) {
      const uint4 q = x8[i8];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int i = i8 * 8 + k;
        // a bf16 is the upper half of the fp32 with the same value
        const float v = __uint_as_float((k & 1) ? (w[k >> 1] & 0xFFFF0000u) : (w[k >> 1] << 16));
        if (i == mask_a || i == mask_b) continue;
        if (v > best || (v == best && i < bidx)) { best = v; bidx = i; }
      }
    }
    for (int i = (V8 << 3) + threadIdx.x; i < V; i += blockDim.x) {
      if (i == mask_a || i == mask_b) continue;
      const float v = ld_logit<T>(x, i);
      if (v > best || (v == best && i < bidx)) { best = v; bidx = i; }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      if (i == mask_a || i == mask_b) continue;
      const float v = ld_logit<T>(x, i);
      if (v > best || (v == best && i < bidx)) { best = v; bidx = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
    if (ov > best || (ov == best && oi < bidx)) { best = ov; bidx = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) { s_val[w] = best; s_idx[w] = bidx; }
  __syncthreads();
  if (w == 0) {
    best = l < nw ? s_val[l] : -INFINITY;
    bidx = l < nw ? s_idx[l] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
      if (ov > best || (ov == best && oi < bidx)) { best = ov; bidx = oi; }
    }
    if (l == 0) { s_val[0] = best; s_idx[0] = bidx; }
  }
  __syncthreads();
  best = s_val[0];
  bidx = s_idx[0];
  if (threadIdx.x == 0) {
    if (pair_out) {
      // vocabulary shard: publish (max logit, global index); the cross-rank merge picks the winner
      pair_out[row] = make_uint2(__float_as_uint(best), (uint32_t)(bidx == 0x7fffffff ? 0x7fffffff : bidx + idx_offset));
    } else {
      if (bidx == 0x7fffffff) bidx = 0;
      const int orow = row_map ? row_map[row] : row;
      out_ids[orow] = bidx;
      if (feed) feed[orow] = bidx;
    }
  }
  if (out_logprob) {
    float se = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) se += __expf(ld_logit<T>(x, i) - best);
    se = mb::block_sum(se, s_red);
    if (threadIdx.x == 0) out_logprob[row_map ? row_map[row] : row] = -__logf(se);
  }
}

struct SampleParams {
  const float* logits;      // [M, ld] fp32 (penalties / bias already applied)
  long long ld;
  int V;
  const float* temperature; // [M]; <= 0 means greedy
  const int* top_k;         // [M]; <= 0 means off
  const float* top_p;       // [M]; >= 1 means off
  const float* min_p;       // [M]; <= 0 means off
  const unsigned long long* seed;  // [M]
  const unsigned long long* step;  // [M]
  int* out_ids;
  float* out_logprob;       // log-prob of the chosen token under the unfiltered softmax
};

__device__ __forceinline__ float u01(unsigned long long seed, unsigned long long ctr) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (ctr + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)((z >> 40) + 0.5) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(1024) sample_kernel(const SampleParams p) {
  __shared__ float s_red[32];
  __shared__ float s_f[4];
  __shared__ int s_i[2];
  __shared__ float s_scan[1024];
  const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
  const float* x = p.logits + (size_t)row * p.ld;
  const int V = p.V;
  const float temp = p.temperature[row];
  // max / argmax
  float best = -INFINITY;
  int bidx = 0x7fffffff;
  for (int i = tid; i < V; i += nt) {
    const float v = x[i];
    if (v > best || (v == best && i < bidx)) { best = v; bidx = i; }
  }
  {
    __shared__ float sv[32];
    __shared__ int si[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
      if (ov > best || (ov == best && oi < bidx)) { best = ov; bidx = oi; }
    }
    if ((tid & 31) == 0) { sv[tid >> 5] = best; si[tid >> 5] = bidx; }
    __syncthreads();
    if (tid < 32) {
      best = tid < (nt >> 5) ? sv[tid] : -INFINITY;
      bidx = tid < (nt >> 5) ? si[tid] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
        if (ov > best || (ov == best && oi < bidx)) { best = ov; bidx = oi; }
      }
      if (tid == 0) { s_f[0] = best; s_i[0] = bidx; }
    }
    __syncthreads();
    best = s_f[0];
    bidx = s_i[0];
  }
  // unfiltered log-sum-exp at temperature 1 (for the reported log-prob)
  float se1 = 0.f;
  for (int i = tid; i < V; i += nt) se1 += __expf(x[i] - best);
  se1 = mb::block_sum(se1, s_red);
  if (!(temp > 0.f)) {
    if (tid == 0) {
      p.out_ids[row] = bidx;
      if (p.out_logprob) p.out_logprob[row] = -__logf(se1);
    }
    return;
  }
  const float invt = 1.f / temp;
  // weights w_i = exp((x_i - max) / T); thresholds live in the logit domain
  uint32_t thr = 0;  // ordered image; keep x with ordered(x) >= thr
  const int k = p.top_k ? p.top_k[row] : 0;
  if (k > 0 && k < V) {
    // largest t with count(ordered(x) >= t) >= k  -> the k-th largest value
    uint32_t lo = 0, hi = 0xFFFFFFFFu;
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1) + 1;
      float c = 0.f;
      for (int i = tid; i < V; i += nt) c += ordered_u32(x[i]) >= mid ? 1.f : 0.f;
      c = mb::block_sum(c, s_red);
      if (c >= (float)k) lo = mid; else hi = mid - 1;
    }
    thr = lo;
  }
  const float mp = p.min_p ? p.min_p[row] : 0.f;
  if (mp > 0.f) {
    const float t = best + temp * __logf(mp);   // w_i >= min_p * w_max
    const uint32_t o = ordered_u32(t);
    if (o > thr) thr = o;
  }
  const float tp = p.top_p ? p.top_p[row] : 1.f;
  if (tp < 1.f) {
    float mass = 0.f;
    for (int i = tid; i < V; i += nt)
      mass += ordered_u32(x[i]) >= thr ? __expf((x[i] - best) * invt) : 0.f;
    mass = mb::block_sum(mass, s_red);
    const float need = tp * mass;
    // largest t >= thr with mass(ordered(x) >= t) >= need
    uint32_t lo = thr, hi = ordered_u32(best);
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1) + 1;
      float c = 0.f;
      for (int i = tid; i < V; i += nt)
        c += ordered_u32(x[i]) >= mid ? __expf((x[i] - best) * invt) : 0.f;
      c = mb::block_sum(c, s_red);
      if (c >= need) lo = mid; else hi = mid - 1;
    }
    thr = lo;
  }
  // multinomial over the kept set, cumulative in index order; each thread owns a
  // contiguous segment so the scan order is the index order
  const int seg = (V + nt - 1) / nt;
  const int i0 = tid * seg, i1 = min(V, i0 + seg);
  float local = 0.f;
  for (int i = i0; i < i1; ++i)
    local += ordered_u32(x[i]) >= thr ? __expf((x[i] - best) * invt) : 0.f;
  s_scan[tid] = local;
  __syncthreads();
  // inclusive scan (Hillis-Steele, nt <= 1024)
  for (int o = 1; o < nt; o <<= 1) {
    const float add = tid >= o ? s_scan[tid - o] : 0.f;
    __syncthreads();
    s_scan[tid] += add;
    __syncthreads();
  }
  const float total = s_scan[nt - 1];
  const float u = u01(p.seed[row], p.step[row]) * total;
  if (tid == 0) s_i[1] = -1;
  __syncthreads();
  const float before = tid == 0 ? 0.f : s_scan[tid - 1];
  if (local > 0.f && u >= before && u < s_scan[tid]) {
    float acc = before;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      if (ordered_u32(x[i]) >= thr) {
        acc += __expf((x[i] - best) * invt);
        pick = i;
        if (u < acc) break;
      }
    }
    s_i[1] = pick;
  }
  __syncthreads();
  if (tid == 0) {
    int pick = s_i[1];
    if (pick < 0) pick = bidx;  // numerical edge: fall back to the mode
    p.out_ids[row] = pick;
    if (p.out_logprob) p.out_logprob[row] = (x[pick] - best) - __logf(se1);
  }
}

// logits[row, tok] adjusted in place from a per-row list of triples.
__global__ void penalties_kernel(float* __restrict__ logits, long long ld, int V,
                                 const int* __restrict__ tok, const int* __restrict__ cnt,
                                 const int* __restrict__ in_prompt, int max_hist,
                                 const float* __restrict__ rep, const float* __restrict__ pres,
                                 const float* __restrict__ freq) {
  const int row = blockIdx.x;
  float* x = logits + (size_t)row * ld;
  const float r = rep ? rep[row] : 1.f, pr = pres ? pres[row] : 0.f, fr = freq ? freq[row] : 0.f;
  for (int j = threadIdx.x; j < max_hist; j += blockDim.x) {
    const int t = tok[(size_t)row * max_hist + j];
    if (t < 0 || t >= V) continue;
    const int c = cnt[(size_t)row * max_hist + j];   // occurrences in the generated text
    const int ip = in_prompt ? in_prompt[(size_t)row * max_hist + j] : 0;
    float v = x[t];
    if (r != 1.f && (c > 0 || ip)) v = v > 0.f ? v / r : v * r;
    if (c > 0) v -= pr + fr * (float)c;
    x[t] = v;
  }
}

}  // namespace

extern "C" {

int mb_argmax(const void* logits, int is_f32, long long ld, int M, int V, int* out_ids,
              float* out_logprob, int mask_a, int mask_b, int* feed, const int* row_map,
              cudaStream_t stream) {
  if (!logits || !out_ids || M <= 0 || V <= 0) return MB_ERR_BAD_ARG;
  if (is_f32)
    argmax_kernel<float><<<M, 1024, 0, stream>>>(reinterpret_cast<const float*>(logits), ld, V,
                                                 out_ids, out_logprob, mask_a, mask_b, feed, row_map,
                                                 nullptr, 0);
  else
    argmax_kernel<__nv_bfloat16><<<M, 1024, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(logits), ld, V, out_ids, out_logprob, mask_a, mask_b,
        feed, row_map, nullptr, 0);
  return (int)cudaGetLastError();
}

// Argmax over one rank's shard of the vocabulary: writes (max logit bits, idx_offset + local
// index) per row into `pairs` (8 bytes per row) for mb_tp_argmax_merge.
int mb_argmax_shard(const void* logits, int is_f32, long long ld, int M, int V, void* pairs,
                    int idx_offset, cudaStream_t stream) {
  if (!logits || !pairs || M <= 0 || V <= 0) return MB_ERR_BAD_ARG;
  if (is_f32)
    argmax_kernel<float><<<M, 1024, 0, stream>>>(reinterpret_cast<const float*>(logits), ld, V, nullptr,
                                                 nullptr, -1, -1, nullptr, nullptr,
                                                 reinterpret_cast<uint2*>(pairs), idx_offset);
  else
    argmax_kernel<__nv_bfloat16><<<M, 1024, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(logits), ld, V, nullptr, nullptr, -1, -1, nullptr, nullptr,
        reinterpret_cast<uint2*>(pairs), idx_offset);
  return (int)cudaGetLastError();
}

int mb_sample(const float* logits, long long ld, int M, int V, const float* temperature,
              const int* top_k, const float* top_p, const float* min_p,
              const unsigned long long* seed, const unsigned long long* step, int* out_ids,
              float* out_logprob, cudaStream_t stream) {
  if (!logits || !temperature || !seed || !step || !out_ids || M <= 0 || V <= 0) return MB_ERR_BAD_ARG;
  SampleParams p{logits, ld, V, temperature, top_k, top_p, min_p, seed, step, out_ids, out_logprob};
  sample_kernel<<<M, 1024, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

int mb_apply_penalties(float* logits, long long ld, int M, int V, const int* tok, const int* cnt,
                       const int* in_prompt, int max_hist, const float* rep, const float* pres,
                       const float* freq, cudaStream_t stream) {
  if (!logits || !tok || !cnt || M <= 0 || max_hist <= 0) return MB_ERR_BAD_ARG;
  penalties_kernel<<<M, 256, 0, stream>>>(logits, ld, V, tok, cnt, in_prompt, max_hist, rep, pres, freq);
  return (int)cudaGetLastError();
}

}  // extern "C"
