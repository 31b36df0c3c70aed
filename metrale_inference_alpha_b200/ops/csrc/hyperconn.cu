// Kernels on the multi-stream fp32 residual "highway" of hyper-connection models: the stream holds
// hc copies [T, hc, H] instead of one row per token; every block reads a learned mixture of the
// copies and writes back through a learned, doubly-stochastic-normalised combination.
//
//   hc_pre    one CTA per token:
//               flat  = streams[t] / sqrt(mean(streams[t]^2) + norm_eps)        over all hc*H values
//               mixes = fn @ flat                              [(2 + hc) * hc] = pre | post | comb
//               pre   = sigmoid(pre * s0 + base) + eps
//               post  = 2 * sigmoid(post * s1 + base)
//               comb  = softmax_j(comb * s2 + base) + eps, one column normalisation, then
//                       (iters - 1) x (row, column) normalisations, each dividing by (sum + eps)
//               y     = sum_i pre[i] * streams[t, i]            (bf16: the block's input)
//             The raw dot products are taken on the un-normalised stream and scaled by the rms
//             factor afterwards, so the stream is read once for both the statistics and the mix.
//   hc_post   out[t, j, :] = post[t, j] * block_out[t, :] + sum_i comb[t, i, j] * streams[t, i, :]
//             (in place: a thread reads all hc values of its column before it writes them)
//   engram_gate_add   streams[t, c, :] += sigmoid(ssqrt(dot)) * value[t, :], with
//             dot = sum_d h[d] qk[c, d] key[t, c, d] * rsqrt(mean(h^2)+eps) * rsqrt(mean(key^2)+eps) / sqrt(H)
//             and ssqrt(x) = sign(x) sqrt(max(|x|, 1e-6))
//   ple_gate  per token: gate[c] = sigmoid(ssqrt(<norm_k(key)[c], norm_q(h)[c]> / sqrt(H))) per stream
//             (grouped RMSNorms with (1 + w) weights), gated[c, :] = gate[c] * value, and its
//             grouped RMSNorm for the following dilated convolution
//   dilated_conv   depthwise causal conv with dilation, SiLU, added to a base tensor; carries
//             (taps - 1) * dilation steps of state per sequence
//
// Reference behaviour covered: kernels/gb10/common/glm5next_mhc.cu (pre / post),
// kernels/gb10/deepseek-v4-flash/nvfp4/{hyper_connection,engram_v41}.cu,
// kernels/gb10/qwen3.8-flash-next/nvfp4/ple.cu.
#include "common.cuh"

namespace {

constexpr int kMaxHc = 4;
constexpr int kMaxMix = (2 + kMaxHc) * kMaxHc;
constexpr int kHcThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = mb::warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
  return t;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float ssqrt(float x) { return copysignf(sqrtf(fmaxf(fabsf(x), 1e-6f)), x); }

// The gates and the combination matrix of one token from its (rms-scaled) mixes, by warp 0: lane = element
// (i, j) = (lane / 4, lane % 4) of the 4 x 4 grid (elements outside hc x hc carry zeros). Row sums meet through
// shuffles over the lanes of a row (xor 1, 2), column sums over xor 4, 8; every normalisation is one reciprocal
// and one multiply per lane, so the Sinkhorn iterations cost a few hundred cycles instead of a serial chain of
// divisions.
__device__ __forceinline__ void hc_gates_warp(const float* mix, float rstd, const float* __restrict__ scale,
                                              const float* __restrict__ base, int hc, float hc_eps, int iters,
                                              float* pre_s, float* post_out, float* comb_out) {
  const int lane = threadIdx.x & 31;
  const int i = (lane >> 2) & 3, j = lane & 3;
  const bool in = lane < 16 && i < hc && j < hc;
  if (lane < hc) {
    pre_s[lane] = sigmoidf_(mix[lane] * rstd * scale[0] + base[lane]) + hc_eps;
    post_out[lane] = 2.f * sigmoidf_(mix[hc + lane] * rstd * scale[1] + base[hc + lane]);
  }
  float c = in ? mix[2 * hc + i * hc + j] * rstd * scale[2] + base[2 * hc + i * hc + j] : -INFINITY;
  float m = fmaxf(c, __shfl_xor_sync(0xffffffffu, c, 1));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
  c = in ? __expf(c - m) : 0.f;
  float rs = c + __shfl_xor_sync(0xffffffffu, c, 1);
  rs += __shfl_xor_sync(0xffffffffu, rs, 2);
  c = in ? c / rs + hc_eps : 0.f;
  for (int it = 0; it < iters; ++it) {
    if (it > 0) {                                                   // row normalisation
      float r = c + __shfl_xor_sync(0xffffffffu, c, 1);
      r += __shfl_xor_sync(0xffffffffu, r, 2);
      c *= 1.f / (r + hc_eps);
    }
    float cs = c + __shfl_xor_sync(0xffffffffu, c, 4);              // column normalisation
    cs += __shfl_xor_sync(0xffffffffu, cs, 8);
    c *= 1.f / (cs + hc_eps);
  }
  if (in) comb_out[i * hc + j] = c;
}

__global__ void __launch_bounds__(kHcThreads)
hc_pre_kernel(const float* __restrict__ streams, const __nv_bfloat16* __restrict__ fn, const float* __restrict__ scale,
              const float* __restrict__ base, __nv_bfloat16* __restrict__ y, float* __restrict__ post_out,
              float* __restrict__ comb_out, int hc, int H, float norm_eps, float hc_eps, int iters) {
  __shared__ float mix[kMaxMix];
  __shared__ float pre_s[kMaxHc];
  const int t = blockIdx.x;
  const int n = hc * H, mix_hc = (2 + hc) * hc;
  const float* x = streams + (size_t)t * n;
  float ss = 0.f, acc[kMaxMix];
#pragma unroll
  for (int r = 0; r < kMaxMix; ++r) acc[r] = 0.f;
  // eight consecutive stream values per step: two 16-byte loads of the stream, one of every mixing row
  const int n8 = (n % 8 == 0) ? n / 8 : 0;
  for (int i8 = threadIdx.x; i8 < n8; i8 += kHcThreads) {
    const float4 x0 = reinterpret_cast<const float4*>(x)[2 * i8], x1 = reinterpret_cast<const float4*>(x)[2 * i8 + 1];
    const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fmaf(xv[j], xv[j], ss);
#pragma unroll
    for (int r = 0; r < kMaxMix; ++r) {
      if (r < mix_hc) {
        const uint4 w = reinterpret_cast<const uint4*>(fn + (size_t)r * n)[i8];
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(w2[j]);
          acc[r] = fmaf(f.x, xv[2 * j], acc[r]);
          acc[r] = fmaf(f.y, xv[2 * j + 1], acc[r]);
        }
      }
    }
  }
  for (int i = n8 * 8 + threadIdx.x; i < n; i += kHcThreads) {
    const float v = x[i];
    ss = fmaf(v, v, ss);
#pragma unroll
    for (int r = 0; r < kMaxMix; ++r)
      if (r < mix_hc) acc[r] = fmaf(__bfloat162float(fn[(size_t)r * n + i]), v, acc[r]);
  }
  // one reduction for the statistic and all mixing rows: warp sums, then kMaxMix + 1 threads add the warps' partials
  __shared__ float part[kMaxMix + 1][kHcThreads / 32];
  ss = mb::warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[kMaxMix][threadIdx.x >> 5] = ss;
#pragma unroll
  for (int r = 0; r < kMaxMix; ++r) {
    if (r < mix_hc) {
      const float v = mb::warp_sum(acc[r]);
      if ((threadIdx.x & 31) == 0) part[r][threadIdx.x >> 5] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x <= kMaxMix && (threadIdx.x < mix_hc || threadIdx.x == kMaxMix)) {
    float v = 0.f;
    for (int w = 0; w < kHcThreads / 32; ++w) v += part[threadIdx.x][w];
    part[threadIdx.x][0] = v;
  }
  __syncthreads();
  if (threadIdx.x < mix_hc) mix[threadIdx.x] = part[threadIdx.x][0] * rsqrtf(part[kMaxMix][0] / n + norm_eps);
  __syncthreads();
  if (threadIdx.x < 32)
    hc_gates_warp(mix, 1.f, scale, base, hc, hc_eps, iters, pre_s, post_out + (size_t)t * hc, comb_out + (size_t)t * hc * hc);
  __syncthreads();
  for (int d = threadIdx.x; d < H; d += kHcThreads) {
    float v = 0.f;
    for (int i = 0; i < hc; ++i) v = fmaf(pre_s[i], x[(size_t)i * H + d], v);
    y[(size_t)t * H + d] = __float2bfloat16(v);
  }
}

// ---- the same computation split for many rows: `hc_mix` walks (4-token tile, slice of the hc*H axis) so that a
// slice of the mixing matrix is read once per four tokens and the grid fills the machine whatever the row count;
// it leaves per-slice partial sums, which `hc_finish` adds in slice order (no atomics: the result does not
// depend on scheduling) before the gates, the Sinkhorn iterations and the collapse.
constexpr int kMixTok = 4, kMixThreads = 64;

__global__ void __launch_bounds__(kMixThreads)
hc_mix_kernel(const float* __restrict__ streams, const __nv_bfloat16* __restrict__ fn, float* __restrict__ part,
              int T, int hc, int H, int slices) {
  __shared__ float red[kMixThreads / 32][kMixTok][kMaxMix + 1];
  const int n = hc * H, mix_hc = (2 + hc) * hc;
  const int t0 = blockIdx.x * kMixTok, sl = blockIdx.y;
  const int n8 = n / 8, per = (n8 + slices - 1) / slices;
  const int lo = sl * per, hi = min(n8, lo + per);
  float acc[kMixTok][kMaxMix], ss[kMixTok];
#pragma unroll
  for (int m = 0; m < kMixTok; ++m) {
    ss[m] = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxMix; ++r) acc[m][r] = 0.f;
  }
  for (int i8 = lo + threadIdx.x; i8 < hi; i8 += kMixThreads) {
    float xv[kMixTok][8];
#pragma unroll
    for (int m = 0; m < kMixTok; ++m) {
      if (t0 + m < T) {
        const float4* xp = reinterpret_cast<const float4*>(streams + (size_t)(t0 + m) * n) + 2 * i8;
        const float4 a = xp[0], b = xp[1];
        xv[m][0] = a.x; xv[m][1] = a.y; xv[m][2] = a.z; xv[m][3] = a.w;
        xv[m][4] = b.x; xv[m][5] = b.y; xv[m][6] = b.z; xv[m][7] = b.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) xv[m][j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss[m] = fmaf(xv[m][j], xv[m][j], ss[m]);
    }
#pragma unroll
    for (int r = 0; r < kMaxMix; ++r) {
      if (r < mix_hc) {
        const uint4 w = reinterpret_cast<const uint4*>(fn + (size_t)r * n)[i8];
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&w);
        float wf[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(w2[j]);
          wf[2 * j] = f.x;
          wf[2 * j + 1] = f.y;
        }
#pragma unroll
        for (int m = 0; m < kMixTok; ++m)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[m][r] = fmaf(wf[j], xv[m][j], acc[m][r]);
      }
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int m = 0; m < kMixTok; ++m) {
    const float s = mb::warp_sum(ss[m]);
    if (lane == 0) red[warp][m][kMaxMix] = s;
#pragma unroll
    for (int r = 0; r < kMaxMix; ++r) {
      if (r < mix_hc) {
        const float v = mb::warp_sum(acc[m][r]);
        if (lane == 0) red[warp][m][r] = v;
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kMixTok * (kMaxMix + 1); i += kMixThreads) {
    const int m = i / (kMaxMix + 1), r = i - m * (kMaxMix + 1);
    if (t0 + m < T && (r < mix_hc || r == kMaxMix)) {
      float v = 0.f;
      for (int w = 0; w < kMixThreads / 32; ++w) v += red[w][m][r];
      part[((size_t)sl * T + t0 + m) * (kMaxMix + 1) + r] = v;
    }
  }
}

__global__ void __launch_bounds__(kHcThreads)
hc_finish_kernel(const float* __restrict__ streams, const float* __restrict__ part, const float* __restrict__ scale,
                 const float* __restrict__ base, __nv_bfloat16* __restrict__ y, float* __restrict__ post_out,
                 float* __restrict__ comb_out, int T, int hc, int H, int slices, float norm_eps, float hc_eps, int iters) {
  __shared__ float mix[kMaxMix + 1];
  __shared__ float pre_s[kMaxHc];
  const int t = blockIdx.x;
  const int n = hc * H, mix_hc = (2 + hc) * hc;
  const float* x = streams + (size_t)t * n;
  if (threadIdx.x <= kMaxMix && (threadIdx.x < mix_hc || threadIdx.x == kMaxMix)) {
    float v = 0.f;
    for (int s = 0; s < slices; ++s) v += part[((size_t)s * T + t) * (kMaxMix + 1) + threadIdx.x];
    mix[threadIdx.x] = v;
  }
  __syncthreads();
  if (threadIdx.x < 32)
    hc_gates_warp(mix, rsqrtf(mix[kMaxMix] / n + norm_eps), scale, base, hc, hc_eps, iters, pre_s,
                  post_out + (size_t)t * hc, comb_out + (size_t)t * hc * hc);
  __syncthreads();
  for (int d = threadIdx.x; d < H; d += kHcThreads) {
    float v = 0.f;
    for (int i = 0; i < hc; ++i) v = fmaf(pre_s[i], x[(size_t)i * H + d], v);
    y[(size_t)t * H + d] = __float2bfloat16(v);
  }
}

__global__ void __launch_bounds__(kHcThreads)
hc_post_kernel(const __nv_bfloat16* __restrict__ block_out, float* __restrict__ streams, const float* __restrict__ post,
               const float* __restrict__ comb, int hc, int H) {
  __shared__ float p[kMaxHc], c[kMaxHc][kMaxHc];
  const int t = blockIdx.x;
  if (threadIdx.x < hc) p[threadIdx.x] = post[(size_t)t * hc + threadIdx.x];
  if (threadIdx.x < hc * hc) c[threadIdx.x / hc][threadIdx.x % hc] = comb[(size_t)t * hc * hc + threadIdx.x];
  __syncthreads();
  float* x = streams + (size_t)t * hc * H;
  for (int d = blockIdx.y * kHcThreads + threadIdx.x; d < H; d += gridDim.y * kHcThreads) {
    const float b = __bfloat162float(block_out[(size_t)t * H + d]);
    float r[kMaxHc], o[kMaxHc];
#pragma unroll
    for (int i = 0; i < kMaxHc; ++i) r[i] = i < hc ? x[(size_t)i * H + d] : 0.f;
#pragma unroll
    for (int j = 0; j < kMaxHc; ++j) {
      float v = j < hc ? p[j] * b : 0.f;
#pragma unroll
      for (int i = 0; i < kMaxHc; ++i)
        if (i < hc && j < hc) v = fmaf(c[i][j], r[i], v);
      o[j] = v;
    }
#pragma unroll
    for (int j = 0; j < kMaxHc; ++j)
      if (j < hc) x[(size_t)j * H + d] = o[j];
  }
}

// grid (T, hc): one CTA per (token, stream)
__global__ void __launch_bounds__(kHcThreads)
engram_gate_add_kernel(float* __restrict__ streams, const __nv_bfloat16* __restrict__ kv, const float* __restrict__ qk,
                       int hc, int H, float eps) {
  __shared__ float red[kHcThreads / 32];
  const int t = blockIdx.x, c = blockIdx.y;
  float* h = streams + ((size_t)t * hc + c) * H;
  const __nv_bfloat16* key = kv + (size_t)t * H * (hc + 1) + (size_t)c * H;
  const __nv_bfloat16* val = kv + (size_t)t * H * (hc + 1) + (size_t)hc * H;
  float sh = 0.f, sk = 0.f, dot = 0.f;
  for (int d = threadIdx.x; d < H; d += kHcThreads) {
    const float hv = h[d], kvv = __bfloat162float(key[d]);
    sh = fmaf(hv, hv, sh);
    sk = fmaf(kvv, kvv, sk);
    dot = fmaf(hv * qk[(size_t)c * H + d], kvv, dot);
  }
  sh = block_sum(sh, red);
  sk = block_sum(sk, red);
  dot = block_sum(dot, red);
  const float g = sigmoidf_(ssqrt(dot * rsqrtf(sh / H + eps) * rsqrtf(sk / H + eps) * rsqrtf((float)H)));
  for (int d = threadIdx.x; d < H; d += kHcThreads) h[d] = fmaf(g, __bfloat162float(val[d]), h[d]);
}

// grid T. key [T, hc*H] bf16, value [T, H] bf16, hidden [T, hc*H] fp32; w_* are (1 + w) RMSNorm weights
// over each stream's H-wide slice. Writes gated [T, hc*H] fp32 and its norm_conv image.
__global__ void __launch_bounds__(kHcThreads)
ple_gate_kernel(const float* __restrict__ hidden, const __nv_bfloat16* __restrict__ key,
                const __nv_bfloat16* __restrict__ value, const float* __restrict__ w_key, const float* __restrict__ w_query,
                const float* __restrict__ w_conv, float* __restrict__ gated, float* __restrict__ normed, int hc, int H,
                float eps) {
  __shared__ float red[kHcThreads / 32];
  const int t = blockIdx.x;
  float sv = 0.f;
  for (int d = threadIdx.x; d < H; d += kHcThreads) {
    const float v = __bfloat162float(value[(size_t)t * H + d]);
    sv = fmaf(v, v, sv);
  }
  sv = block_sum(sv, red);
  for (int c = 0; c < hc; ++c) {
    const float* h = hidden + ((size_t)t * hc + c) * H;
    const __nv_bfloat16* k = key + ((size_t)t * hc + c) * H;
    float sh = 0.f, sk = 0.f, dot = 0.f;
    for (int d = threadIdx.x; d < H; d += kHcThreads) {
      const float hv = h[d], kvv = __bfloat162float(k[d]);
      sh = fmaf(hv, hv, sh);
      sk = fmaf(kvv, kvv, sk);
      dot = fmaf(hv * (1.f + w_query[(size_t)c * H + d]), kvv * (1.f + w_key[(size_t)c * H + d]), dot);
    }
    sh = block_sum(sh, red);
    sk = block_sum(sk, red);
    dot = block_sum(dot, red);
    const float g = sigmoidf_(ssqrt(dot * rsqrtf(sh / H + eps) * rsqrtf(sk / H + eps) * rsqrtf((float)H)));
    // the gated value of this stream is g * value, so its mean square is g^2 * mean(value^2)
    const float rstd = rsqrtf(g * g * sv / H + eps);
    for (int d = threadIdx.x; d < H; d += kHcThreads) {
      const float gv = g * __bfloat162float(value[(size_t)t * H + d]);
      gated[((size_t)t * hc + c) * H + d] = gv;
      normed[((size_t)t * hc + c) * H + d] = gv * rstd * (1.f + w_conv[(size_t)c * H + d]);
    }
  }
}

// out[t, ch] = base[t, ch] + silu(sum_j w[ch, j] * x[t - (taps - 1 - j) * dil, ch]); inputs before the
// sequence start come from state [slots, C, (taps-1)*dil] (zero for a fresh sequence), which is
// advanced by the sequence's rows afterwards. grid (ceil(C / 256), sequences).
__global__ void __launch_bounds__(256)
dilated_conv_kernel(const float* __restrict__ x, const float* __restrict__ basep, const float* __restrict__ w,
                    float* __restrict__ state, float* __restrict__ out, int C, int taps, int dil,
                    const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ positions,
                    const int* __restrict__ slots, int num_slots, int write_state, uint32_t* status) {
  const int ch = blockIdx.x * blockDim.x + threadIdx.x, seq = blockIdx.y;
  const int n = q_len[seq];
  if (ch >= C || n <= 0) return;
  const int slot = slots[seq];
  if (slot < 0 || slot >= num_slots) {
    if (status) atomicCAS(status, 0u, MB_ST_BOUNDS);
    return;
  }
  const int q0 = q_start[seq], hist = (taps - 1) * dil;
  const bool fresh = positions[q0] == 0;
  float* st = state + ((size_t)slot * C + ch) * hist;
  float wv[8];
  for (int j = 0; j < taps; ++j) wv[j] = w[(size_t)ch * taps + j];
  for (int t = 0; t < n; ++t) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = (taps - 1 - j) * dil, src = t - back;
      float v;
      if (src >= 0) v = x[(size_t)(q0 + src) * C + ch];
      else v = fresh ? 0.f : st[hist + src];                        // st[hist - 1] is the newest kept input
      acc = fmaf(wv[j], v, acc);
    }
    out[(size_t)(q0 + t) * C + ch] = basep[(size_t)(q0 + t) * C + ch] + acc / (1.f + __expf(-acc));
  }
  if (write_state) {
    // new history = the last `hist` inputs of (old history ++ this call's rows)
    float keep[16];
    for (int i = 0; i < hist; ++i) {
      const int src = n - hist + i;                                 // index into this call's rows
      keep[i] = src >= 0 ? x[(size_t)(q0 + src) * C + ch] : (fresh ? 0.f : st[hist + src]);
    }
    for (int i = 0; i < hist; ++i) st[i] = keep[i];
  }
}

}  // namespace

extern "C" int mb_hc_pre_ws_floats(int T, int hc, int H) {
  // slices chosen so that (token tiles x slices) covers the machine about twice
  const int tiles = (T + kMixTok - 1) / kMixTok;
  int slices = (296 + tiles - 1) / tiles;
  const int n8 = hc * H / 8;
  if (slices > n8 / kMixThreads) slices = n8 / kMixThreads;
  if (slices < 1) slices = 1;
  if (slices > 32) slices = 32;
  return slices * T * (kMaxMix + 1);
}

extern "C" int mb_hc_pre_split(const void* streams, const void* fn, const void* scale, const void* base, void* y,
                               void* post, void* comb, void* ws, int ws_floats, int T, int hc, int H, float norm_eps,
                               float hc_eps, int iters, cudaStream_t stream) {
  if (!streams || !fn || !y || !ws || T <= 0 || hc <= 0 || hc > kMaxHc || H <= 0 || iters < 1 || (hc * H) % 8)
    return MB_ERR_BAD_ARG;
  const int need = mb_hc_pre_ws_floats(T, hc, H);
  if (ws_floats < need) return MB_ERR_TOO_LARGE;
  const int slices = need / (T * (kMaxMix + 1));
  hc_mix_kernel<<<dim3((T + kMixTok - 1) / kMixTok, slices), kMixThreads, 0, stream>>>(
      static_cast<const float*>(streams), static_cast<const __nv_bfloat16*>(fn), static_cast<float*>(ws), T, hc, H, slices);
  hc_finish_kernel<<<T, kHcThreads, 0, stream>>>(
      static_cast<const float*>(streams), static_cast<const float*>(ws), static_cast<const float*>(scale),
      static_cast<const float*>(base), static_cast<__nv_bfloat16*>(y), static_cast<float*>(post),
      static_cast<float*>(comb), T, hc, H, slices, norm_eps, hc_eps, iters);
  return (int)cudaGetLastError();
}

extern "C" int mb_hc_pre(const void* streams, const void* fn, const void* scale, const void* base, void* y, void* post,
                         void* comb, int T, int hc, int H, float norm_eps, float hc_eps, int iters, cudaStream_t stream) {
  if (!streams || !fn || !y || T <= 0 || hc <= 0 || hc > kMaxHc || H <= 0 || iters < 1) return MB_ERR_BAD_ARG;
  hc_pre_kernel<<<T, kHcThreads, 0, stream>>>(static_cast<const float*>(streams), static_cast<const __nv_bfloat16*>(fn),
                                              static_cast<const float*>(scale), static_cast<const float*>(base),
                                              static_cast<__nv_bfloat16*>(y), static_cast<float*>(post),
                                              static_cast<float*>(comb), hc, H, norm_eps, hc_eps, iters);
  return (int)cudaGetLastError();
}

extern "C" int mb_hc_post(const void* block_out, void* streams, const void* post, const void* comb, int T, int hc, int H,
                          cudaStream_t stream) {
  if (!block_out || !streams || T <= 0 || hc <= 0 || hc > kMaxHc) return MB_ERR_BAD_ARG;
  const int by = (H + kHcThreads * 4 - 1) / (kHcThreads * 4);
  hc_post_kernel<<<dim3(T, by < 1 ? 1 : by), kHcThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(block_out), static_cast<float*>(streams), static_cast<const float*>(post),
      static_cast<const float*>(comb), hc, H);
  return (int)cudaGetLastError();
}

extern "C" int mb_engram_gate_add(void* streams, const void* kv, const void* qk, int T, int hc, int H, float eps,
                                  cudaStream_t stream) {
  if (!streams || !kv || !qk || T <= 0 || hc <= 0) return MB_ERR_BAD_ARG;
  engram_gate_add_kernel<<<dim3(T, hc), kHcThreads, 0, stream>>>(
      static_cast<float*>(streams), static_cast<const __nv_bfloat16*>(kv), static_cast<const float*>(qk), hc, H, eps);
  return (int)cudaGetLastError();
}

extern "C" int mb_ple_gate(const void* hidden, const void* key, const void* value, const void* w_key, const void* w_query,
                           const void* w_conv, void* gated, void* normed, int T, int hc, int H, float eps,
                           cudaStream_t stream) {
  if (!hidden || !key || !value || !gated || !normed || T <= 0 || hc <= 0) return MB_ERR_BAD_ARG;
  ple_gate_kernel<<<T, kHcThreads, 0, stream>>>(
      static_cast<const float*>(hidden), static_cast<const __nv_bfloat16*>(key), static_cast<const __nv_bfloat16*>(value),
      static_cast<const float*>(w_key), static_cast<const float*>(w_query), static_cast<const float*>(w_conv),
      static_cast<float*>(gated), static_cast<float*>(normed), hc, H, eps);
  return (int)cudaGetLastError();
}

extern "C" int mb_dilated_conv(const void* x, const void* base, const void* w, void* state, void* out, int C, int taps,
                               int dil, const void* q_start, const void* q_len, const void* positions, const void* slots,
                               int num_seqs, int num_slots, int write_state, void* status, cudaStream_t stream) {
  if (!x || !base || !w || !state || !out || C <= 0 || taps < 1 || taps > 8 || dil < 1 || (taps - 1) * dil > 16 ||
      num_seqs <= 0)
    return MB_ERR_BAD_ARG;
  dilated_conv_kernel<<<dim3((C + 255) / 256, num_seqs), 256, 0, stream>>>(
      static_cast<const float*>(x), static_cast<const float*>(base), static_cast<const float*>(w),
      static_cast<float*>(state), static_cast<float*>(out), C, taps, dil, static_cast<const int*>(q_start),
      static_cast<const int*>(q_len), static_cast<const int*>(positions), static_cast<const int*>(slots), num_slots,
      write_state, static_cast<uint32_t*>(status));
  return (int)cudaGetLastError();
}
