// GGUF block formats -> bf16 on the device, so a llama.cpp checkpoint is uploaded in its packed form
// (a quarter to a half of the bf16 bytes over PCIe) and widened where the bandwidth is.
//
// One thread per 8 output values (one 16-byte store), grid-stride free: the launch covers exactly
// nblocks * values-per-block / 8 threads. Block layouts as in ggml:
//   Q8_0  32 values: f16 d | 32 x i8                              value = d * q
//   Q4_0  32 values: f16 d | 16 bytes (j: low nibble, j + 16: high) value = d * (q - 8)
//   Q4_K  256 values: f16 d, f16 dmin | 12 bytes of 6-bit scales / mins | 128 bytes
//         group g of 64: 32 low nibbles with (scale, min) 2g, 32 high nibbles with 2g + 1
//   Q6_K  256 values: 128 bytes ql | 64 bytes qh | 16 x i8 scales | f16 d; value = d * scale * (q - 32)
// The host implementation in weights/gguf.py is the oracle.
//
// Reference behaviour covered: the GGUF GPU dequantisation kernels of the reference's loader
// (crates/model-weights GGUF container + GPU dequant, kernels/gb10/common dequant family).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int kQ8_0 = 8, kQ4_0 = 2, kQ4_K = 12, kQ6_K = 14;

__device__ __forceinline__ float f16_at(const uint8_t* p) {
  const uint16_t b = (uint16_t)p[0] | ((uint16_t)p[1] << 8);
  return __half2float(__ushort_as_half(b));
}
__device__ __forceinline__ void store8(__nv_bfloat16* dst, const float (&v)[8]) {
  uint4 o;
  __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
  *reinterpret_cast<uint4*>(dst) = o;
}

__global__ void q8_0_kernel(const uint8_t* __restrict__ raw, __nv_bfloat16* __restrict__ out, long long nblocks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;      // 4 threads per block
  if (i >= nblocks * 4) return;
  const uint8_t* b = raw + (i >> 2) * 34;
  const float d = f16_at(b);
  const int8_t* q = reinterpret_cast<const int8_t*>(b + 2) + (i & 3) * 8;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = d * (float)q[j];
  store8(out + i * 8, v);
}

__global__ void q4_0_kernel(const uint8_t* __restrict__ raw, __nv_bfloat16* __restrict__ out, long long nblocks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;      // 4 threads per block
  if (i >= nblocks * 4) return;
  const uint8_t* b = raw + (i >> 2) * 18;
  const float d = f16_at(b);
  const int part = (int)(i & 3);                                              // values part*8 .. part*8+7
  const uint8_t* qs = b + 2 + (part & 1) * 8;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int q = part < 2 ? (qs[j] & 0x0F) : (qs[j] >> 4);
    v[j] = d * (float)(q - 8);
  }
  store8(out + i * 8, v);
}

__global__ void q4_k_kernel(const uint8_t* __restrict__ raw, __nv_bfloat16* __restrict__ out, long long nblocks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;      // 32 threads per block
  if (i >= nblocks * 32) return;
  const uint8_t* b = raw + (i >> 5) * 144;
  const int t = (int)(i & 31);                 // values t*8 .. t*8+7
  const int g = t >> 3;                        // group of 64
  const int hi = (t >> 2) & 1;                 // second half of the group: high nibbles
  const int j = 2 * g + hi;                    // (scale, min) index
  const uint8_t* sc = b + 4;
  int s, m;
  if (j < 4) { s = sc[j] & 63; m = sc[j + 4] & 63; }
  else { s = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4); m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
  const float d = f16_at(b) * (float)s, mn = f16_at(b + 2) * (float)m;
  const uint8_t* qs = b + 16 + g * 32 + (t & 3) * 8;
  float v[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = d * (float)(hi ? (qs[k] >> 4) : (qs[k] & 0x0F)) - mn;
  store8(out + i * 8, v);
}

__global__ void q6_k_kernel(const uint8_t* __restrict__ raw, __nv_bfloat16* __restrict__ out, long long nblocks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;      // 32 threads per block
  if (i >= nblocks * 32) return;
  const uint8_t* b = raw + (i >> 5) * 210;
  const int t = (int)(i & 31);                 // values t*8 .. t*8+7
  const int half = t >> 4, quarter = (t >> 2) & 3, off = (t & 3) * 8;         // 128 / 32 / 8 values
  const uint8_t* ql = b + half * 64 + (quarter & 1) * 32 + off;
  const uint8_t* qh = b + 128 + half * 32 + off;
  const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192) + half * 8 + quarter * 2 + (off >> 4);
  const float d = f16_at(b + 208) * (float)sc[0];
  float v[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int lo = quarter < 2 ? (ql[k] & 0x0F) : (ql[k] >> 4);
    const int h = (qh[k] >> (2 * quarter)) & 3;
    v[k] = d * (float)((lo | (h << 4)) - 32);
  }
  store8(out + i * 8, v);
}

}  // namespace

// raw: device copy of the tensor's block bytes; out: bf16 [nblocks * values per block] (16-byte aligned).
// Returns 0, 1 for an unsupported type, or 100 + the CUDA error.
extern "C" int mb_gguf_dequant(int type, const void* raw, long long nblocks, void* out, cudaStream_t st) {
  if (nblocks <= 0) return 0;
  const uint8_t* r = (const uint8_t*)raw;
  __nv_bfloat16* o = (__nv_bfloat16*)out;
  const int threads = 256;
  const long long per = (type == kQ4_K || type == kQ6_K) ? 32 : 4;
  const unsigned blocks = (unsigned)((nblocks * per + threads - 1) / threads);
  if (type == kQ8_0) q8_0_kernel<<<blocks, threads, 0, st>>>(r, o, nblocks);
  else if (type == kQ4_0) q4_0_kernel<<<blocks, threads, 0, st>>>(r, o, nblocks);
  else if (type == kQ4_K) q4_k_kernel<<<blocks, threads, 0, st>>>(r, o, nblocks);
  else if (type == kQ6_K) q6_k_kernel<<<blocks, threads, 0, st>>>(r, o, nblocks);
  else return 1;
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 100 + (int)e;
}
