// Weight-only-quantised linears with bf16 activations ("W4A16" for NVFP4 weights, "W8A16" for
// FP8 weights): the activation is used exactly as the previous layer produced it, only the weight
// is low precision. Two kernels:
//
//   a16_gemv_kernel   out[m, n] = sum_k x[m, k] * dequant(W[n, k]) for up to 8 rows of x. It is a
//                     streaming kernel: each warp owns two weight rows (a gate / up pair when the
//                     SwiGLU epilogue is on), every lane reads 32 NVFP4 or 16 FP8 weights per step with
//                     one 16-byte load, widens them in registers and accumulates in fp32
//                     against the activation rows staged in shared memory. One pass over the
//                     packed weights; the host loops row blocks of 8 for a few more rows.
//   a16_dequant_kernel  widens a row band of the weight to bf16 so that the tensor-core bf16 GEMM
//                     serves large M (prefill), where one extra pass over the weights is amortised
//                     over hundreds of activation rows.
//
// Same role as the reference's NVFP4- / FP8-weight GEMMs with bf16 activations
// (kernels/gb10/common/w4a16_gemm.cu:3-15, w4a16_gemv.cu, w8a16_gemv.cu, w8a16_gemm.cu), which
// tile the same contraction for mma.sync on another architecture.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int kKindFp8Row = 1, kKindNvfp4 = 2, kKindFp8Block = 3;
constexpr int kChunk = 2048;          // K values of x staged per pass
constexpr int kWarps = 8;

struct A16Params {
  const uint8_t* W;         // fp8: [N, K]; nvfp4: [N, K/2]
  const void* scale;        // fp8_row: f32 [N]; fp8_block: f32 [ceil(N/128), ceil(K/128)]; nvfp4: e4m3 [N, K/16]
  const float* row_gscale;  // nvfp4: optional per-row global scale
  float gscale;             // nvfp4: global scale
  const __nv_bfloat16* x;   // [M, ldx]
  const __nv_bfloat16* residual;   // [M, ldo] or null
  __nv_bfloat16* out;       // [M, ldo]
  float* out_f32;           // used instead of `out` when not null
  int M, N, K, ldx, ldo, swiglu, scale_ld;
};

__device__ __forceinline__ void widen8_fp8(uint2 w, float (&v)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t word = (i < 2) ? w.x : w.y;
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((word >> (16 * (i & 1))) & 0xFFFF), __NV_E4M3);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void widen8_fp4(uint32_t w, float (&v)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)((w >> (8 * i)) & 0xFF), __NV_E2M1);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
    v[2 * i] = f.x;       // low nibble = even k
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// Values of one weight row a lane consumes per step: one 16-byte load (32 NVFP4 nibbles or 16 FP8
// bytes). A warp step then covers 32 * kVpl consecutive k. The staged activations are stored
// lane-interleaved, [step][8-value group j][lane][8], so that the 16-byte shared-memory reads of a
// warp are consecutive (no bank conflicts) although each lane's k range is contiguous in global memory.
template <int KIND> struct Vpl { static constexpr int v = KIND == kKindNvfp4 ? 32 : 16; };

template <int KIND, int MT>
__global__ void __launch_bounds__(kWarps * 32) a16_gemv_kernel(const A16Params p) {
  constexpr int kVpl = Vpl<KIND>::v, kJ = kVpl / 8, kStepK = 32 * kVpl;
  __shared__ __align__(16) __nv_bfloat16 xs[MT][kChunk];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * kWarps + warp) * 2;
  float acc[2][MT];
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
  const size_t wld = KIND == kKindNvfp4 ? (size_t)p.K / 2 : (size_t)p.K;

  for (int k0 = 0; k0 < p.K; k0 += kChunk) {
    __syncthreads();
    for (int i = threadIdx.x; i < MT * (kChunk / 8); i += kWarps * 32) {
      const int m = i / (kChunk / 8), c = (i % (kChunk / 8)) * 8;          // c: offset of an 8-value group in the chunk
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < p.M && k0 + c < p.K) v = *reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx + k0 + c);
      const int step = c / kStepK, in = c % kStepK, ln = in / kVpl, jj = (in % kVpl) / 8;
      *reinterpret_cast<uint4*>(&xs[m][step * kStepK + jj * 256 + ln * 8]) = v;
    }
    __syncthreads();
    if (n0 >= p.N) continue;
#pragma unroll 2
    for (int s = 0; s < kChunk / kStepK; ++s) {
      const int k = k0 + s * kStepK + lane * kVpl;
      if (k >= p.K) break;
      uint4 wq[2];
      float ws[2][2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int n = min(n0 + r, p.N - 1);
        if (KIND == kKindNvfp4) {
          wq[r] = *reinterpret_cast<const uint4*>(p.W + n * wld + k / 2);
          const uint16_t sf2 = *reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(p.scale) + (size_t)n * (p.K / 16) + k / 16);
          ws[r][0] = e4m3_to_float((uint8_t)(sf2 & 0xFF));
          ws[r][1] = e4m3_to_float((uint8_t)(sf2 >> 8));
        } else {
          wq[r] = *reinterpret_cast<const uint4*>(p.W + n * wld + k);
          ws[r][0] = ws[r][1] = KIND == kKindFp8Block
                                    ? reinterpret_cast<const float*>(p.scale)[(size_t)(n / 128) * p.scale_ld + k / 128]
                                    : 1.f;
        }
      }
#pragma unroll
      for (int jj = 0; jj < kJ; ++jj) {
        float wv[2][8];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const uint32_t* w32 = reinterpret_cast<const uint32_t*>(&wq[r]);
          if (KIND == kKindNvfp4) widen8_fp4(w32[jj], wv[r]);
          else widen8_fp8(make_uint2(w32[2 * jj], w32[2 * jj + 1]), wv[r]);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const uint4 xv = *reinterpret_cast<const uint4*>(&xs[m][s * kStepK + jj * 256 + lane * 8]);
          const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xv);
          float xf[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(xb[i]);
            xf[2 * i] = f.x;
            xf[2 * i + 1] = f.y;
          }
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) d = fmaf(wv[r][i], xf[i], d);
            acc[r][m] = fmaf(d, ws[r][KIND == kKindNvfp4 ? jj / 2 : 0], acc[r][m]);
          }
        }
      }
    }
  }
  if (n0 >= p.N) return;
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[r][m] += __shfl_xor_sync(0xffffffffu, acc[r][m], o);
  if (lane != 0) return;
  float rs[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int n = min(n0 + r, p.N - 1);
    if (KIND == kKindFp8Row) rs[r] = reinterpret_cast<const float*>(p.scale)[n];
    else if (KIND == kKindNvfp4) rs[r] = p.gscale * (p.row_gscale ? p.row_gscale[n] : 1.f);
    else rs[r] = 1.f;
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    if (m >= p.M) break;
    if (p.swiglu) {
      const float g = acc[0][m] * rs[0], u = acc[1][m] * rs[1];
      const float y = g / (1.f + __expf(-g)) * u;
      const size_t o = (size_t)m * p.ldo + n0 / 2;
      if (p.out_f32) p.out_f32[o] = y; else p.out[o] = __float2bfloat16(y);
    } else {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (n0 + r >= p.N) break;
        const size_t o = (size_t)m * p.ldo + n0 + r;
        float y = acc[r][m] * rs[r];
        if (p.residual) y += __bfloat162float(p.residual[o]);
        if (p.out_f32) p.out_f32[o] = y; else p.out[o] = __float2bfloat16(y);
      }
    }
  }
}

// rows [n_lo, n_lo + rows) of the weight -> bf16 [rows, K]; one thread widens 8 values
template <int KIND>
__global__ void a16_dequant_kernel(const A16Params p, int n_lo, int rows, __nv_bfloat16* dst) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int per_row = p.K / 8;
  if (i >= (size_t)rows * per_row) return;
  const int n = n_lo + (int)(i / per_row), k = (int)(i % per_row) * 8;
  float v[8], s;
  if (KIND == kKindNvfp4) {
    widen8_fp4(*reinterpret_cast<const uint32_t*>(p.W + (size_t)n * (p.K / 2) + k / 2), v);
    s = e4m3_to_float(reinterpret_cast<const uint8_t*>(p.scale)[(size_t)n * (p.K / 16) + k / 16]) * p.gscale *
        (p.row_gscale ? p.row_gscale[n] : 1.f);
  } else {
    widen8_fp8(*reinterpret_cast<const uint2*>(p.W + (size_t)n * p.K + k), v);
    s = KIND == kKindFp8Block ? reinterpret_cast<const float*>(p.scale)[(size_t)(n / 128) * p.scale_ld + k / 128]
                              : reinterpret_cast<const float*>(p.scale)[n];
  }
  uint4 o;
  __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(v[2 * j] * s, v[2 * j + 1] * s);
  *reinterpret_cast<uint4*>(dst + (size_t)(n - n_lo) * p.K + k) = o;
}

template <int KIND>
cudaError_t launch_gemv(const A16Params& p, cudaStream_t st) {
  const int blocks = (p.N + 2 * kWarps - 1) / (2 * kWarps);
  if (p.M <= 1) a16_gemv_kernel<KIND, 1><<<blocks, kWarps * 32, 0, st>>>(p);
  else if (p.M <= 2) a16_gemv_kernel<KIND, 2><<<blocks, kWarps * 32, 0, st>>>(p);
  else if (p.M <= 4) a16_gemv_kernel<KIND, 4><<<blocks, kWarps * 32, 0, st>>>(p);
  else a16_gemv_kernel<KIND, 8><<<blocks, kWarps * 32, 0, st>>>(p);
  return cudaGetLastError();
}

}  // namespace

struct MbA16Args {
  int kind, M, N, K, ldx, ldo, swiglu, scale_ld;
  const void* W;
  const void* scale;
  const void* row_gscale;
  const void* x;
  const void* residual;
  void* out;
  void* out_f32;
  float gscale;
  int n_lo, rows;           // dequant only
};

static int fill(const MbA16Args* a, A16Params& p) {
  if (a->K % 32 != 0 || a->ldx % 8 != 0 || (a->swiglu && (a->N & 1))) return 1;
  if (a->kind != kKindFp8Row && a->kind != kKindNvfp4 && a->kind != kKindFp8Block) return 1;
  p.W = (const uint8_t*)a->W; p.scale = a->scale; p.row_gscale = (const float*)a->row_gscale;
  p.gscale = a->gscale; p.x = (const __nv_bfloat16*)a->x; p.residual = (const __nv_bfloat16*)a->residual;
  p.out = (__nv_bfloat16*)a->out; p.out_f32 = (float*)a->out_f32;
  p.M = a->M; p.N = a->N; p.K = a->K; p.ldx = a->ldx; p.ldo = a->ldo; p.swiglu = a->swiglu; p.scale_ld = a->scale_ld;
  return 0;
}

// Up to 8 activation rows against the packed weight. Returns 0, 1 (bad argument) or a CUDA error + 100.
extern "C" int mb_a16_gemv(const MbA16Args* a, cudaStream_t st) {
  A16Params p;
  if (fill(a, p) || a->M < 1 || a->M > 8) return 1;
  cudaError_t e = a->kind == kKindNvfp4 ? launch_gemv<kKindNvfp4>(p, st)
                : a->kind == kKindFp8Row ? launch_gemv<kKindFp8Row>(p, st) : launch_gemv<kKindFp8Block>(p, st);
  return e == cudaSuccess ? 0 : 100 + (int)e;
}

// Rows [n_lo, n_lo + rows) of the weight as bf16 [rows, K] into a->out.
extern "C" int mb_a16_dequant(const MbA16Args* a, cudaStream_t st) {
  A16Params p;
  if (fill(a, p) || a->rows < 1 || a->n_lo < 0 || a->n_lo + a->rows > a->N) return 1;
  const size_t total = (size_t)a->rows * (a->K / 8);
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  __nv_bfloat16* dst = (__nv_bfloat16*)a->out;
  if (a->kind == kKindNvfp4) a16_dequant_kernel<kKindNvfp4><<<blocks, threads, 0, st>>>(p, a->n_lo, a->rows, dst);
  else if (a->kind == kKindFp8Row) a16_dequant_kernel<kKindFp8Row><<<blocks, threads, 0, st>>>(p, a->n_lo, a->rows, dst);
  else a16_dequant_kernel<kKindFp8Block><<<blocks, threads, 0, st>>>(p, a->n_lo, a->rows, dst);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 100 + (int)e;
}
