// Batched multi-adapter LoRA ("BGMV"): every token row carries an adapter slot (-1 = none) and
//     out[m, n0 + n] += scale[a] * sum_r B[a][n][r] * (sum_k A[a][r][k] * x[m][k])
// in two launches: shrink (x -> rank-r vector per row, fp32) and expand-fold (add into the bf16
// output of the base projection, at a column offset so fused q|k|v outputs can be addressed).
// Rows with slot -1 cost one predicate. Rank <= 64. These are decode-sized ops (a few rows x
// rank), CUDA-core dot products; the base projection stays on the tensor cores.
// Reference behaviour: kernels/gb10/common/lora_bgmv.cu (lora_bgmv_shrink, lora_bgmv_expand_fold).
#include "common.cuh"

namespace {

constexpr int kMaxRank = 64;

// grid (M), 256 threads: warp w computes ranks w, w + 8, ...
__global__ void lora_shrink_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ A,
                                   const int* __restrict__ slots, float* __restrict__ tmp, int K, int rank,
                                   int num_slots, uint32_t* status) {
  const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int a = slots[m];
  if (a < 0) return;
  if (a >= num_slots) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0u, MB_ST_BOUNDS);
    return;
  }
  const __nv_bfloat16* xr = x + (size_t)m * ldx;
  for (int r = warp; r < rank; r += 8) {
    const __nv_bfloat16* ar = A + ((size_t)a * rank + r) * K;
    float acc = 0.f;
    for (int k = lane * 8; k + 8 <= K; k += 256) {
      const uint4 xv = *reinterpret_cast<const uint4*>(xr + k);
      const uint4 av = __ldg(reinterpret_cast<const uint4*>(ar + k));
      const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xv);
      const __nv_bfloat162* ab = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 xf = __bfloat1622float2(xb[i]), af = __bfloat1622float2(ab[i]);
        acc += xf.x * af.x + xf.y * af.y;
      }
    }
    for (int k = (K & ~7) + lane; k < K; k += 32) acc += __bfloat162float(xr[k]) * __bfloat162float(ar[k]);
    acc = mb::warp_sum(acc);
    if (lane == 0) tmp[(size_t)m * kMaxRank + r] = acc;
  }
}

// grid (M, ceil(N / 256)), 256 threads: one output column per thread
__global__ void lora_expand_kernel(const float* __restrict__ tmp, const __nv_bfloat16* __restrict__ B,
                                   const int* __restrict__ slots, const float* __restrict__ scales,
                                   __nv_bfloat16* __restrict__ out, int ldo, int n0, int N, int rank, int num_slots) {
  const int m = blockIdx.x, n = blockIdx.y * 256 + threadIdx.x;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int a = slots[m];
  if (a < 0 || a >= num_slots) return;
  __shared__ float s_t[kMaxRank];
  if (threadIdx.x < rank) s_t[threadIdx.x] = tmp[(size_t)m * kMaxRank + threadIdx.x] * scales[a];
  __syncthreads();
  if (n >= N) return;
  const __nv_bfloat16* br = B + ((size_t)a * N + n) * rank;
  float acc = 0.f;
  for (int r = 0; r < rank; ++r) acc += s_t[r] * __bfloat162float(br[r]);
  __nv_bfloat16* o = out + (size_t)m * ldo + n0 + n;
  *o = __float2bfloat16(__bfloat162float(*o) + acc);
}

}  // namespace

extern "C" {

// x [M, K] bf16 (row stride ldx); A [num_slots, rank, K] bf16; tmp [M, 64] fp32
int mb_lora_shrink(const void* x, int ldx, const void* A, const int* slots, float* tmp, int M, int K, int rank,
                   int num_slots, uint32_t* status, cudaStream_t stream) {
  if (!x || !A || !slots || !tmp || M <= 0 || K <= 0 || rank <= 0 || rank > kMaxRank || (ldx % 8) || (K % 8 && false))
    return MB_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(A)) & 15) return MB_ERR_BAD_ARG;
  if (K % 8) return MB_ERR_UNSUPPORTED;
  return (int)mb::launch_kernel(lora_shrink_kernel, dim3(M), dim3(256), (size_t)0, stream,
                                reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<const __nv_bfloat16*>(A),
                                slots, tmp, K, rank, num_slots, status);
}

// B [num_slots, N, rank] bf16; out [M, ldo] bf16, columns n0 .. n0 + N receive the delta
int mb_lora_expand(const float* tmp, const void* B, const int* slots, const float* scales, void* out, int ldo, int n0,
                   int M, int N, int rank, int num_slots, cudaStream_t stream) {
  if (!tmp || !B || !slots || !scales || !out || M <= 0 || N <= 0 || rank <= 0 || rank > kMaxRank) return MB_ERR_BAD_ARG;
  return (int)mb::launch_kernel(lora_expand_kernel, dim3(M, (N + 255) / 256), dim3(256), (size_t)0, stream, tmp,
                                reinterpret_cast<const __nv_bfloat16*>(B), slots, scales,
                                reinterpret_cast<__nv_bfloat16*>(out), ldo, n0, N, rank, num_slots);
}

}  // extern "C"
