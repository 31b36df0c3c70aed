// Row-wise fused producer kernels: one CTA owns one token row, builds the fp32
// row in shared memory from one of several "input" recipes and writes it in one
// of several "output" encodings, so normalisation / activation / quantisation
// never make a separate trip through HBM.
//
// input recipes
//   IN_COPY          y = x
//   IN_RMSNORM       h = x (+ residual); residual_out = bf16(h);
//                    y = h * rsqrt(mean(h^2) + eps) * (w | 1 + w)
//   IN_SILU_MUL      y = silu(x[:, k]) * x[:, K + k]        (x is [M, 2K], gate | up)
//   IN_RELU2         y = relu(x)^2
//   IN_SIGMOID_GATE  y = x * sigmoid(gate), gate addressed per head with strides
//   IN_GATED_RMSNORM y = rmsnorm_group(x) * w * silu(gate)   (GDN / Mamba2 output norm;
//                    statistics over groups of `group` channels)
// output encodings
//   OUT_BF16         bf16 [M, K]
//   OUT_FP8_ROW      e4m3 [M, K] + scale[M] = amax / 448
//   OUT_FP8_G128     e4m3 [M, K] + scale[K/128][ld] per token per 128 channels
//   OUT_NVFP4        packed e2m1 [M, K/2] + ue4m3 scale factors in the 128x4 tiled
//                    layout tcgen05.cp consumes + per-token fp32 scale amax/(6*448)
// `also_bf16` additionally writes the bf16 row (router / MTP consumers).
//
// Reference behaviour covered: kernels/gb10/common/rms_norm.cu (rms_norm,
// residual_add_rms_norm, gated_rms_norm), rms_norm_act_quant.cu, moe_silu_mul.cu,
// relu_squared.cu, residual_add.cu::sigmoid_gate_mul, quantize_bf16_to_nvfp4.cu,
// w8a8_act_quant.cu, per_token_group_quant_fp8.
#include "common.cuh"
#include <cstdlib>

namespace {

enum { IN_COPY = 0, IN_RMSNORM = 1, IN_SILU_MUL = 2, IN_RELU2 = 3, IN_SIGMOID_GATE = 4,
       IN_GATED_RMSNORM = 5 };
enum { OUT_BF16 = 0, OUT_FP8_ROW = 1, OUT_FP8_G128 = 2, OUT_NVFP4 = 3 };

struct RowParams {
  int M, K;
  int in_mode, out_mode;
  const __nv_bfloat16* x;
  long long x_ld;
  const __nv_bfloat16* residual;      // [M, K] or null
  __nv_bfloat16* residual_out;        // [M, K] or null
  const __nv_bfloat16* w;             // norm weight [K] or null
  int w_plus_one;
  float eps;
  const __nv_bfloat16* gate;          // IN_SIGMOID_GATE / IN_GATED_RMSNORM
  long long gate_ld;
  int head_dim, gate_head_stride, gate_head_off;
  int group;                          // IN_GATED_RMSNORM statistics group (0 = whole row)
  const float* xf32;                  // optional fp32 input instead of x (GDN core output)
  void* out;
  long long out_ld;                   // in elements of the output encoding (bytes for fp8/fp4)
  __nv_bfloat16* out_bf16;            // also_bf16 target or null
  long long out_bf16_ld;
  float* scale;                       // per-token scale(s)
  int scale_ld;                       // OUT_FP8_G128: tokens stride
  uint8_t* sf;                        // OUT_NVFP4 tiled scale factors
  int sf_k64;
  float static_gs;                    // OUT_NVFP4: > 0 = calibrated global scale instead of the row's amax / (6 * 448)
  const int* row_index;               // optional [M]: CTA i works on row row_index[i] (negative: none) instead of row i
};

__device__ __forceinline__ float load_x(const RowParams& p, int m, int k) {
  if (p.xf32) return p.xf32[(size_t)m * p.x_ld + k];
  return __bfloat162float(p.x[(size_t)m * p.x_ld + k]);
}

__global__ void __launch_bounds__(512) row_kernel(const RowParams p) {
  extern __shared__ float row[];
  __shared__ float red[32];
  const int K = p.K;
  const int tid = threadIdx.x, nt = blockDim.x;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int m = p.row_index ? p.row_index[blockIdx.x] : (int)blockIdx.x;
  if (m < 0) return;

  // ---- stage 1: build the fp32 row
  if (p.in_mode == IN_RMSNORM) {
    float ss = 0.f;
    for (int k = tid; k < K; k += nt) {
      float h = load_x(p, m, k);
      if (p.residual) {
        h += __bfloat162float(p.residual[(size_t)m * K + k]);
        h = __bfloat162float(__float2bfloat16(h));
      }
      if (p.residual_out) p.residual_out[(size_t)m * K + k] = __float2bfloat16(h);
      row[k] = h;
      ss += h * h;
    }
    ss = mb::block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)K + p.eps);
    for (int k = tid; k < K; k += nt) {
      float w = p.w ? __bfloat162float(p.w[k]) : 1.f;
      if (p.w_plus_one) w += 1.f;
      row[k] = row[k] * inv * w;
    }
  } else if (p.in_mode == IN_GATED_RMSNORM) {
    const int G = p.group > 0 ? p.group : K;
    for (int k = tid; k < K; k += nt) row[k] = load_x(p, m, k);
    __syncthreads();
    // one warp per statistics group
    const int warp = tid >> 5, lane = tid & 31, nw = nt >> 5;
    for (int g = warp; g * G < K; g += nw) {
      float ss = 0.f;
      for (int k = lane; k < G; k += 32) { const float v = row[g * G + k]; ss += v * v; }
      ss = mb::warp_sum(ss);
      const float inv = rsqrtf(ss / (float)G + p.eps);
      for (int k = lane; k < G; k += 32) {
        const int kk = g * G + k;
        const float w = p.w ? __bfloat162float(p.w[kk]) : 1.f;
        float y = row[kk] * inv * w;
        if (p.gate) y *= mb::silu(__bfloat162float(p.gate[(size_t)m * p.gate_ld + kk]));
        row[kk] = y;
      }
    }
  } else {
    for (int k = tid; k < K; k += nt) {
      float y;
      if (p.in_mode == IN_SILU_MUL) {
        const float g = load_x(p, m, k), u = load_x(p, m, K + k);
        y = mb::silu(g) * u;
      } else if (p.in_mode == IN_RELU2) {
        const float v = fmaxf(load_x(p, m, k), 0.f);
        y = v * v;
      } else if (p.in_mode == IN_SIGMOID_GATE) {
        const int h = k / p.head_dim, d = k - h * p.head_dim;
        const float g = __bfloat162float(
            p.gate[(size_t)m * p.gate_ld + (size_t)h * p.gate_head_stride + p.gate_head_off + d]);
        y = load_x(p, m, k) / (1.f + __expf(-g));
      } else {
        y = load_x(p, m, k);
      }
      row[k] = y;
    }
  }
  __syncthreads();

  if (p.out_bf16) {
    for (int k = tid; k < K; k += nt)
      p.out_bf16[(size_t)m * p.out_bf16_ld + k] = __float2bfloat16(row[k]);
  }

  // ---- stage 2: encode
  if (p.out_mode == OUT_BF16) {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.out_ld;
    for (int k = tid; k < K; k += nt) o[k] = __float2bfloat16(row[k]);
  } else if (p.out_mode == OUT_FP8_ROW) {
    float amax = 0.f;
    for (int k = tid; k < K; k += nt) amax = fmaxf(amax, fabsf(row[k]));
    amax = mb::block_max(amax, red);
    const float sc = amax > 0.f ? amax / 448.f : 1.f;
    const float inv = 1.f / sc;
    if (tid == 0) p.scale[m] = sc;
    uint8_t* o = reinterpret_cast<uint8_t*>(p.out) + (size_t)m * p.out_ld;
    for (int k = tid; k < K; k += nt) o[k] = mb::float_to_e4m3(row[k] * inv);
  } else if (p.out_mode == OUT_FP8_G128) {
    const int warp = tid >> 5, lane = tid & 31, nw = nt >> 5;
    uint8_t* o = reinterpret_cast<uint8_t*>(p.out) + (size_t)m * p.out_ld;
    for (int g = warp; g * 128 < K; g += nw) {
      float v[4];
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k = g * 128 + lane * 4 + i;
        v[i] = k < K ? row[k] : 0.f;
        amax = fmaxf(amax, fabsf(v[i]));
      }
      amax = mb::warp_max(amax);
      const float sc = amax > 0.f ? amax / 448.f : 1.f;
      const float inv = 1.f / sc;
      if (lane == 0) p.scale[(size_t)g * p.scale_ld + m] = sc;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k = g * 128 + lane * 4 + i;
        if (k < K) o[k] = mb::float_to_e4m3(v[i] * inv);
      }
    }
  } else {  // OUT_NVFP4
    float amax = 0.f;
    for (int k = tid; k < K; k += nt) amax = fmaxf(amax, fabsf(row[k]));
    amax = mb::block_max(amax, red);
    const float gs = p.static_gs > 0.f ? p.static_gs : (amax > 0.f ? amax / (6.f * 448.f) : 1.f);
    if (tid == 0) p.scale[m] = gs;
    uint8_t* o = reinterpret_cast<uint8_t*>(p.out) + (size_t)m * p.out_ld;
    uint8_t* sf_blk = p.sf + (size_t)(m >> 7) * p.sf_k64 * 512;
    const int r = m & 127;
    // one thread per 16-element block
    for (int b = tid; b * 16 < K; b += nt) {
      float v[16];
      float bmax = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int k = b * 16 + i;
        v[i] = k < K ? row[k] : 0.f;
        bmax = fmaxf(bmax, fabsf(v[i]));
      }
      const uint8_t sfc = mb::float_to_e4m3(bmax / (6.f * gs));
      const float sff = mb::e4m3_to_float(sfc);
      const float inv = sff > 0.f ? 1.f / (sff * gs) : 0.f;
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) lo |= mb::e2m1_code(v[i] * inv) << (4 * i);
#pragma unroll
      for (int i = 0; i < 8; ++i) hi |= mb::e2m1_code(v[8 + i] * inv) << (4 * i);
      *reinterpret_cast<uint2*>(o + b * 8) = make_uint2(lo, hi);
      sf_blk[(size_t)(b >> 2) * 512 + mb::sf_tile_offset(r, b & 3)] = sfc;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Fast path for the hot recipes (copy / RMSNorm / SiLU-mul from bf16 rows): every thread owns
// whole 16-element blocks in registers (BPT of them), all global traffic is 16-byte vectors,
// and the row statistics (sum of squares and max |x * w|) share ONE block reduction, so the
// kernel is load -> reduce -> store. amax(y) is taken as max|x w| * inv_rms.
template <int BPT>
__global__ void __launch_bounds__(1024) row_kernel_v2(const RowParams p) {
  __shared__ float red[64];
  const int tid = threadIdx.x, nt = blockDim.x;
  const int K = p.K, nblk = K >> 4;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int m = p.row_index ? p.row_index[blockIdx.x] : (int)blockIdx.x;
  if (m < 0) return;
  float x[BPT][16];
  float ss = 0.f, mx = 0.f;
  const bool norm = p.in_mode == IN_RMSNORM;
#pragma unroll
  for (int j = 0; j < BPT; ++j) {
    const int b = tid + j * nt;
    if (b < nblk) {
      const __nv_bfloat16* src = p.x + (size_t)m * p.x_ld + b * 16;
      uint4 v0 = __ldg(reinterpret_cast<const uint4*>(src));
      uint4 v1 = __ldg(reinterpret_cast<const uint4*>(src) + 1);
      const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&v0);
      const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&v1);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = __bfloat1622float2(h0[i]), c = __bfloat1622float2(h1[i]);
        x[j][2 * i] = a.x; x[j][2 * i + 1] = a.y; x[j][8 + 2 * i] = c.x; x[j][8 + 2 * i + 1] = c.y;
      }
      if (p.in_mode == IN_SILU_MUL) {
        const __nv_bfloat16* up = src + K;
        uint4 u0 = __ldg(reinterpret_cast<const uint4*>(up));
        uint4 u1 = __ldg(reinterpret_cast<const uint4*>(up) + 1);
        const __nv_bfloat162* g0 = reinterpret_cast<const __nv_bfloat162*>(&u0);
        const __nv_bfloat162* g1 = reinterpret_cast<const __nv_bfloat162*>(&u1);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 a = __bfloat1622float2(g0[i]), c = __bfloat1622float2(g1[i]);
          x[j][2 * i] = mb::silu(x[j][2 * i]) * a.x; x[j][2 * i + 1] = mb::silu(x[j][2 * i + 1]) * a.y;
          x[j][8 + 2 * i] = mb::silu(x[j][8 + 2 * i]) * c.x; x[j][8 + 2 * i + 1] = mb::silu(x[j][8 + 2 * i + 1]) * c.y;
        }
      }
      if (norm) {
        float w[16];
        if (p.w) {
          uint4 w0 = __ldg(reinterpret_cast<const uint4*>(p.w + b * 16));
          uint4 w1 = __ldg(reinterpret_cast<const uint4*>(p.w + b * 16) + 1);
          const __nv_bfloat162* q0 = reinterpret_cast<const __nv_bfloat162*>(&w0);
          const __nv_bfloat162* q1 = reinterpret_cast<const __nv_bfloat162*>(&w1);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 a = __bfloat1622float2(q0[i]), c = __bfloat1622float2(q1[i]);
            w[2 * i] = a.x; w[2 * i + 1] = a.y; w[8 + 2 * i] = c.x; w[8 + 2 * i + 1] = c.y;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) w[i] = 1.f;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          ss += x[j][i] * x[j][i];
          x[j][i] *= p.w_plus_one ? (w[i] + 1.f) : w[i];      // x now holds x * w
        }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) mx = fmaxf(mx, fabsf(x[j][i]));
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) x[j][i] = 0.f;
    }
  }
  // one block reduction for (sum of squares, max)
  const bool need_red = norm || p.out_mode == OUT_FP8_ROW || p.out_mode == OUT_NVFP4;
  float inv = 1.f, amax = mx;
  if (need_red) {
    ss = mb::warp_sum(ss);
    mx = mb::warp_max(mx);
    const int w = tid >> 5, l = tid & 31, nw = (nt + 31) >> 5;
    if (l == 0) { red[w] = ss; red[32 + w] = mx; }
    __syncthreads();
    float a = l < nw ? red[l] : 0.f, c = l < nw ? red[32 + l] : 0.f;
    a = mb::warp_sum(a);
    c = mb::warp_max(c);
    if (norm) inv = rsqrtf(a / (float)K + p.eps);
    amax = c * inv;
  }
  float gs = 1.f, row_inv = 1.f;
  if (p.out_mode == OUT_FP8_ROW) {
    gs = amax > 0.f ? amax / 448.f : 1.f;
    row_inv = 1.f / gs;
    if (tid == 0) p.scale[m] = gs;
  } else if (p.out_mode == OUT_NVFP4) {
    gs = p.static_gs > 0.f ? p.static_gs : (amax > 0.f ? amax / (6.f * 448.f) : 1.f);
    if (tid == 0) p.scale[m] = gs;
  }
#pragma unroll
  for (int j = 0; j < BPT; ++j) {
    const int b = tid + j * nt;
    const bool valid = b < nblk;                       // no early exit: the group shuffles below need whole warps
    float y[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) y[i] = x[j][i] * inv;
    if (valid && (p.out_bf16 || p.out_mode == OUT_BF16)) {
      uint4 o0, o1;
      __nv_bfloat162* q0 = reinterpret_cast<__nv_bfloat162*>(&o0);
      __nv_bfloat162* q1 = reinterpret_cast<__nv_bfloat162*>(&o1);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        q0[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
        q1[i] = __floats2bfloat162_rn(y[8 + 2 * i], y[8 + 2 * i + 1]);
      }
      if (p.out_bf16) {
        uint4* d = reinterpret_cast<uint4*>(p.out_bf16 + (size_t)m * p.out_bf16_ld + b * 16);
        d[0] = o0; d[1] = o1;
      }
      if (p.out_mode == OUT_BF16) {
        uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.out_ld + b * 16);
        d[0] = o0; d[1] = o1;
      }
    }
    if (p.out_mode == OUT_FP8_ROW || p.out_mode == OUT_FP8_G128) {
      float sc_inv = row_inv;
      if (p.out_mode == OUT_FP8_G128) {
        float bm = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) bm = fmaxf(bm, fabsf(y[i]));
        // a 128-channel group is 8 consecutive blocks = 8 consecutive lanes
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 4));
        const float sc = bm > 0.f ? bm / 448.f : 1.f;
        sc_inv = 1.f / sc;
        if (valid && (b & 7) == 0) p.scale[(size_t)(b >> 3) * p.scale_ld + m] = sc;
      }
      uint32_t w4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        w4[i] = (uint32_t)mb::float_to_e4m3(y[4 * i] * sc_inv) | ((uint32_t)mb::float_to_e4m3(y[4 * i + 1] * sc_inv) << 8) |
                ((uint32_t)mb::float_to_e4m3(y[4 * i + 2] * sc_inv) << 16) | ((uint32_t)mb::float_to_e4m3(y[4 * i + 3] * sc_inv) << 24);
      }
      if (valid)
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.out) + (size_t)m * p.out_ld + b * 16) =
            make_uint4(w4[0], w4[1], w4[2], w4[3]);
    } else if (p.out_mode == OUT_NVFP4) {
      float bmax = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(y[i]));
      const uint8_t sfc = mb::float_to_e4m3(bmax / (6.f * gs));
      const float sff = mb::e4m3_to_float(sfc);
      const float qi = sff > 0.f ? 1.f / (sff * gs) : 0.f;
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) lo |= mb::e2m1x2_pack(y[2 * i] * qi, y[2 * i + 1] * qi) << (8 * i);
#pragma unroll
      for (int i = 0; i < 4; ++i) hi |= mb::e2m1x2_pack(y[8 + 2 * i] * qi, y[8 + 2 * i + 1] * qi) << (8 * i);
      if (valid)
        *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(p.out) + (size_t)m * p.out_ld + b * 8) = make_uint2(lo, hi);
      uint8_t* sf_blk = p.sf + (size_t)(m >> 7) * p.sf_k64 * 512;
      if ((nblk & 3) == 0) {
        // four consecutive blocks sit on four consecutive lanes and fill one 4-byte group of the tiled
        // scale-factor layout: one 32-bit store per group instead of four byte stores
        const uint32_t s1 = __shfl_down_sync(0xffffffffu, (uint32_t)sfc, 1);
        const uint32_t s2 = __shfl_down_sync(0xffffffffu, (uint32_t)sfc, 2);
        const uint32_t s3 = __shfl_down_sync(0xffffffffu, (uint32_t)sfc, 3);
        if (valid && (b & 3) == 0)
          *reinterpret_cast<uint32_t*>(sf_blk + (size_t)(b >> 2) * 512 + mb::sf_tile_offset(m & 127, 0)) =
              (uint32_t)sfc | (s1 << 8) | (s2 << 16) | (s3 << 24);
      } else if (valid) {
        sf_blk[(size_t)(b >> 2) * 512 + mb::sf_tile_offset(m & 127, b & 3)] = sfc;
      }
    }
  }
}

template <int BPT>
int launch_row_v2(const RowParams& p, int threads, cudaStream_t stream) {
  return (int)mb::launch_kernel(row_kernel_v2<BPT>, dim3(p.M), dim3(threads), 0, stream, p);
}

// Repack row-major ue4m3 scale factors [N, K/16] into the tiled layout
// [ceil(N/128)][sf_k64][512] (zero padded).
__global__ void sf_repack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int N,
                                 int kblocks, int sf_k64) {
  const long long total = (long long)((N + 127) / 128) * sf_k64 * 512;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int within = (int)(i % 512);
    const long long chunk = i / 512;
    const int k64 = (int)(chunk % sf_k64);
    const int nb = (int)(chunk / sf_k64);
    const int kk = within & 3, rq = (within >> 2) & 3, r32 = within >> 4;
    const int r = nb * 128 + rq * 32 + r32;
    const int kb = k64 * 4 + kk;
    dst[i] = (r < N && kb < kblocks) ? src[(size_t)r * kblocks + kb] : 0;
  }
}

// bf16 elementwise add in place: dst += src (2-rank all-reduce tail).
__global__ void add_inplace_kernel(__nv_bfloat16* dst, const __nv_bfloat16* src, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16(__bfloat162float(dst[i]) + __bfloat162float(src[i]));
}

// Token embedding gather: out[m, :] = table[ids[m], :]; ids outside the table give zeros
// and set the status word (no out-of-bounds read).
__global__ void embed_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                             __nv_bfloat16* __restrict__ out, int hidden, int vocab,
                             uint32_t* status) {
  const int m = blockIdx.x;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int id = ids[m];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0 && status) atomicCAS(status, 0u, MB_ST_BOUNDS);
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)(ok ? id : 0) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)m * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x)
    dst[i] = ok ? src[i] : make_uint4(0, 0, 0, 0);
}

}  // namespace

extern "C" {

static int g_pdl = -1;
int mb_pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("METRALE_PDL");
    g_pdl = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 2;   // default: GEMMs launch programmatically   
  }
  return g_pdl;
}
void mb_set_pdl(int mode) { g_pdl = mode < 0 ? 0 : (mode > 2 ? 2 : mode); }

struct MbRowArgs {
  int M, K, in_mode, out_mode;
  const void* x;
  long long x_ld;
  const void* residual;
  void* residual_out;
  const void* w;
  int w_plus_one;
  float eps;
  const void* gate;
  long long gate_ld;
  int head_dim, gate_head_stride, gate_head_off, group;
  const float* xf32;
  void* out;
  long long out_ld;
  void* out_bf16;
  long long out_bf16_ld;
  float* scale;
  int scale_ld;
  void* sf;
  int sf_k64;
  float static_gs;
  const int* row_index;
};

int mb_row_op(const MbRowArgs* a, cudaStream_t stream) {
  if (!a || a->M <= 0 || a->K <= 0 || (!a->x && !a->xf32) || !a->out) return MB_ERR_BAD_ARG;
  if (a->K > 48 * 1024) return MB_ERR_TOO_LARGE;
  if (a->out_mode == OUT_NVFP4 && (a->K % 16 || !a->sf || !a->scale || a->sf_k64 * 64 < a->K))
    return MB_ERR_BAD_ARG;
  if ((a->out_mode == OUT_FP8_ROW || a->out_mode == OUT_FP8_G128) && !a->scale)
    return MB_ERR_BAD_ARG;
  if (a->in_mode == IN_SIGMOID_GATE && (!a->gate || a->head_dim <= 0)) return MB_ERR_BAD_ARG;
  RowParams p{};
  p.M = a->M; p.K = a->K; p.in_mode = a->in_mode; p.out_mode = a->out_mode;
  p.x = reinterpret_cast<const __nv_bfloat16*>(a->x); p.x_ld = a->x_ld;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a->residual);
  p.residual_out = reinterpret_cast<__nv_bfloat16*>(a->residual_out);
  p.w = reinterpret_cast<const __nv_bfloat16*>(a->w); p.w_plus_one = a->w_plus_one;
  p.eps = a->eps;
  p.gate = reinterpret_cast<const __nv_bfloat16*>(a->gate); p.gate_ld = a->gate_ld;
  p.head_dim = a->head_dim; p.gate_head_stride = a->gate_head_stride;
  p.gate_head_off = a->gate_head_off; p.group = a->group;
  p.xf32 = a->xf32;
  p.out = a->out; p.out_ld = a->out_ld;
  p.out_bf16 = reinterpret_cast<__nv_bfloat16*>(a->out_bf16); p.out_bf16_ld = a->out_bf16_ld;
  p.scale = a->scale; p.scale_ld = a->scale_ld;
  p.sf = reinterpret_cast<uint8_t*>(a->sf); p.sf_k64 = a->sf_k64;
  p.static_gs = a->static_gs;
  p.row_index = a->row_index;
  {
    // fast path eligibility: bf16 input, whole 16-element blocks, 16-byte aligned vectors
    const bool modes = p.in_mode == IN_COPY || p.in_mode == IN_RMSNORM || p.in_mode == IN_SILU_MUL;
    const uintptr_t al = reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.out) |
                         reinterpret_cast<uintptr_t>(p.out_bf16) | reinterpret_cast<uintptr_t>(p.w);
    const bool ld_ok = p.x_ld % 8 == 0 && p.out_ld % 8 == 0 && p.out_bf16_ld % 8 == 0;
    const int nblk = a->K / 16;
    if (modes && !p.xf32 && !p.residual && !p.residual_out && a->K % 16 == 0 && !(al & 15) && ld_ok &&
        (p.out_mode != OUT_FP8_G128 || a->K % 128 == 0) && nblk <= 4096) {
      const int bpt = (nblk + 511) / 512;
      int threads = ((nblk + bpt - 1) / bpt + 31) / 32 * 32;
      if (p.out_mode == OUT_FP8_G128) threads = (threads + 7) / 8 * 8;
      switch (bpt) {
        case 1: return launch_row_v2<1>(p, threads, stream);
        case 2: return launch_row_v2<2>(p, threads, stream);
        case 3: return launch_row_v2<3>(p, threads, stream);
        case 4: return launch_row_v2<4>(p, threads, stream);
        default: break;
      }
    }
  }
  const size_t smem = (size_t)a->K * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         48 * 1024 * 4);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int threads = a->K >= 4096 ? 512 : (a->K >= 1024 ? 256 : 128);
  return (int)mb::launch_kernel(row_kernel, dim3(a->M), dim3(threads), smem, stream, p);
}

int mb_sf_repack(const void* src, void* dst, int N, int kblocks, int sf_k64, cudaStream_t stream) {
  if (!src || !dst || N <= 0 || kblocks <= 0 || sf_k64 * 4 < kblocks) return MB_ERR_BAD_ARG;
  const long long total = (long long)((N + 127) / 128) * sf_k64 * 512;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  sf_repack_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(src),
                                               reinterpret_cast<uint8_t*>(dst), N, kblocks, sf_k64);
  return (int)cudaGetLastError();
}

int mb_add_inplace(void* dst, const void* src, long long n, cudaStream_t stream) {
  if (!dst || !src || n <= 0) return MB_ERR_BAD_ARG;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  add_inplace_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(dst),
                                                 reinterpret_cast<const __nv_bfloat16*>(src), n);
  return (int)cudaGetLastError();
}

int mb_embed(const int* ids, const void* table, void* out, int M, int hidden, int vocab,
             uint32_t* status, cudaStream_t stream) {
  if (!ids || !table || !out || M <= 0 || hidden % 8) return MB_ERR_BAD_ARG;
  return (int)mb::launch_kernel(embed_kernel, dim3(M), dim3(128), 0, stream, ids,
                                reinterpret_cast<const __nv_bfloat16*>(table),
                                reinterpret_cast<__nv_bfloat16*>(out), hidden, vocab, status);
}

}  // extern "C"
