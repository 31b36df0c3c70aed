// Chunked (parallel-in-time) prefill scans for the recurrent mixers: long prompts no longer walk
// their tokens one by one.
//
//   mb_mamba2_ssd   Mamba2 selective scan in state-space-dual form, chunk = 64 tokens.
//                   With la_t = -exp(A_log) dt_t and cum_i the inclusive sum of la inside a chunk:
//                     y_i = exp(cum_i) C_i h_start^T + sum_{j<=i} exp(cum_i - cum_j) (C_i . B_j) dt_j x_j + D x_i
//                     h_end = exp(cum_last) h_start + sum_j exp(cum_last - cum_j) dt_j x_j (x) B_j
//                   Three launches for the whole ragged batch:
//                     ssd_chunk_state  per (chunk, head, seq): the chunk's own contribution to the
//                                      state, X_w^T B (64 x 128, K = 64), on the tensor cores;
//                     ssd_state_scan   per (head, seq): the short recurrence over chunks; leaves
//                                      every chunk's start state in the workspace and the final
//                                      state in the pool;
//                     ssd_chunk_out    per (chunk, head, seq): C B^T (64 x 64, K = 128), the
//                                      decay / causal mask, (.) X, and C h_start^T, all three
//                                      products on the tensor cores.
//                   Products run as TF32 `mma.sync.m16n8k8` with fp32 accumulation: the chunk
//                   operands are fp32 activations (conv + SiLU outputs), and a 64-row chunk is
//                   below the 128-row tile at which tcgen05 pays for its TMEM round trip.
//
// The sequential kernels in recurrent.cu stay the oracle and serve decode / verify rows; the
// hand-off state of the chunked path equals theirs to TF32 rounding.
//
// Reference behaviour covered: kernels/gb10/common/mamba2_ssd_chunk.cu (cumsum, bmm and scan
// grids), crates/model-layers Mamba2 prefill.
#include "common.cuh"

namespace {

constexpr int kQ = 64;      // chunk length
constexpr int kP = 64;      // head dim
constexpr int kN = 128;     // state dim

struct SsdParams {
  const float* xbc;          // [T, inner + 2 G N] fp32: x | B | C
  const __nv_bfloat16* dt;   // [T, dt_ld] raw
  long long dt_ld;
  const float* A_log;
  const float* Dp;
  const float* dt_bias;
  float* state;              // [slots, H, P, N]
  float* out;                // [T, H * P]
  float* ws_state;           // [S, max_chunks, H, P * N]: chunk contribution, then chunk start state
  float* ws_decay;           // [S, max_chunks, H]: exp(sum of la over the chunk)
  const int* q_start;
  const int* q_len;
  const int* positions;
  const int* state_slots;
  int H, G, num_slots, max_chunks, write_state;
  uint32_t* status;
};

__device__ __forceinline__ uint32_t to_tf32(float f) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(f));
  return r;
}
__device__ __forceinline__ void mma_tf32(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Per-token gates of one chunk: dtv = softplus(dt + bias), la = -exp(A_log) dtv, inclusive
// prefix sum of la. Tokens past the sequence end get dtv = 0 (they contribute nothing).
// Threads 0..63 each own one token; the result is in s_dtv / s_cum after the barrier.
__device__ __forceinline__ void chunk_gates(const SsdParams& p, int tok0, int valid, int hd, float a_exp,
                                            float* s_dtv, float* s_cum, float* s_tmp) {
  const int tid = threadIdx.x;
  if (tid < kQ) {
    float dtv = 0.f;
    if (tid < valid) {
      const float raw = __bfloat162float(p.dt[(size_t)(tok0 + tid) * p.dt_ld + hd]) + p.dt_bias[hd];
      dtv = raw > 20.f ? raw : log1pf(__expf(raw));
    }
    float v = -a_exp * dtv;
    const int lane = tid & 31;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += n;
    }
    s_dtv[tid] = dtv;
    s_cum[tid] = v;
    if (tid == 31) s_tmp[0] = v;
  }
  __syncthreads();
  if (tid >= 32 && tid < kQ) s_cum[tid] += s_tmp[0];
  __syncthreads();
}

// ------------------------------------------------------------------ chunk state contribution
// S_c[p][n] = sum_j (exp(cum_last - cum_j) dtv_j x_j[p]) B_j[n]
constexpr int kLdX = kP + 8;     // read as [k][m]: stride = 8 (mod 32) keeps the 32 lanes on 32 banks
constexpr int kLdBn = kN + 8;    // read as [k][n]
__global__ void __launch_bounds__(128) ssd_chunk_state_kernel(const SsdParams p) {
  extern __shared__ float sm[];
  float* sX = sm;                         // [kQ][kLdX]   x_j * w_j
  float* sB = sX + kQ * kLdX;             // [kQ][kLdBn]
  float* s_dtv = sB + kQ * kLdBn;
  float* s_cum = s_dtv + kQ;
  float* s_tmp = s_cum + kQ;
  const int c = blockIdx.x, hd = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int n = p.q_len[seq];
  if (c * kQ >= n) return;
  const int tok0 = p.q_start[seq] + c * kQ;
  const int valid = min(kQ, n - c * kQ);
  const int inner = p.H * kP, GN = p.G * kN, ld = inner + 2 * GN;
  const int grp = hd / (p.H / p.G);
  const float a_exp = __expf(p.A_log[hd]);
  chunk_gates(p, tok0, valid, hd, a_exp, s_dtv, s_cum, s_tmp);
  const float cum_last = s_cum[kQ - 1];
  for (int i = tid; i < kQ * (kP / 4); i += 128) {
    const int j = i / (kP / 4), q4 = i - j * (kP / 4);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < valid) {
      v = *reinterpret_cast<const float4*>(p.xbc + (size_t)(tok0 + j) * ld + hd * kP + q4 * 4);
      const float w = __expf(cum_last - s_cum[j]) * s_dtv[j];
      v.x *= w; v.y *= w; v.z *= w; v.w *= w;
    }
    *reinterpret_cast<float4*>(sX + j * kLdX + q4 * 4) = v;
  }
  for (int i = tid; i < kQ * (kN / 4); i += 128) {
    const int j = i / (kN / 4), q4 = i - j * (kN / 4);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < valid) v = *reinterpret_cast<const float4*>(p.xbc + (size_t)(tok0 + j) * ld + inner + grp * kN + q4 * 4);
    *reinterpret_cast<float4*>(sB + j * kLdBn + q4 * 4) = v;
  }
  __syncthreads();
  // warp w owns rows p = 16 w .. 16 w + 15 of the 64 x 128 result; K = 64 tokens
  const int g = lane >> 2, t = lane & 3;
  float acc[kN / 8][4];
#pragma unroll
  for (int nt = 0; nt < kN / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
  const int m0 = warp * 16;
#pragma unroll 2
  for (int k0 = 0; k0 < kQ; k0 += 8) {
    const uint32_t a0 = to_tf32(sX[(k0 + t) * kLdX + m0 + g]);
    const uint32_t a1 = to_tf32(sX[(k0 + t) * kLdX + m0 + g + 8]);
    const uint32_t a2 = to_tf32(sX[(k0 + t + 4) * kLdX + m0 + g]);
    const uint32_t a3 = to_tf32(sX[(k0 + t + 4) * kLdX + m0 + g + 8]);
#pragma unroll
    for (int nt = 0; nt < kN / 8; ++nt) {
      const uint32_t b0 = to_tf32(sB[(k0 + t) * kLdBn + nt * 8 + g]);
      const uint32_t b1 = to_tf32(sB[(k0 + t + 4) * kLdBn + nt * 8 + g]);
      mma_tf32(acc[nt], a0, a1, a2, a3, b0, b1);
    }
  }
  float* dst = p.ws_state + (((size_t)seq * p.max_chunks + c) * p.H + hd) * (kP * kN);
#pragma unroll
  for (int nt = 0; nt < kN / 8; ++nt) {
    *reinterpret_cast<float2*>(dst + (m0 + g) * kN + nt * 8 + 2 * t) = make_float2(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<float2*>(dst + (m0 + g + 8) * kN + nt * 8 + 2 * t) = make_float2(acc[nt][2], acc[nt][3]);
  }
  if (tid == 0) p.ws_decay[((size_t)seq * p.max_chunks + c) * p.H + hd] = __expf(cum_last);
}

// ------------------------------------------------------------------ recurrence over chunks
// grid (H, S), 256 threads, 32 state elements per thread. In place: the workspace slot of
// chunk c receives the state at the START of chunk c.
__global__ void __launch_bounds__(256) ssd_state_scan_kernel(const SsdParams p) {
  const int hd = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int n = p.q_len[seq];
  if (n <= 0) return;
  const int slot = p.state_slots[seq];
  if (slot < 0 || slot >= p.num_slots) {
    if (p.status && tid == 0) atomicCAS(p.status, 0u, MB_ST_BOUNDS);
    return;
  }
  const bool fresh = p.positions[p.q_start[seq]] == 0;
  float* hs = p.state + ((size_t)slot * p.H + hd) * (kP * kN);
  constexpr int kPer = kP * kN / 256;
  float h[kPer];
#pragma unroll
  for (int i = 0; i < kPer; ++i) h[i] = fresh ? 0.f : hs[i * 256 + tid];
  const int chunks = (n + kQ - 1) / kQ;
  for (int c = 0; c < chunks; ++c) {
    float* w = p.ws_state + (((size_t)seq * p.max_chunks + c) * p.H + hd) * (kP * kN);
    const float dec = p.ws_decay[((size_t)seq * p.max_chunks + c) * p.H + hd];
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const float contrib = w[i * 256 + tid];
      w[i * 256 + tid] = h[i];
      h[i] = dec * h[i] + contrib;
    }
  }
  if (p.write_state) {
#pragma unroll
    for (int i = 0; i < kPer; ++i) hs[i * 256 + tid] = h[i];
  }
}

// ------------------------------------------------------------------ chunk outputs
constexpr int kLdC = kN + 4;     // read as [m][k] (and B / h as [n][k]): stride = 4 (mod 32)
constexpr int kLdM = kQ + 4;
__global__ void __launch_bounds__(128) ssd_chunk_out_kernel(const SsdParams p) {
  extern __shared__ float sm[];
  float* sC = sm;                         // [kQ][kLdC]
  float* sB = sC + kQ * kLdC;             // [kQ][kLdC]
  float* sH = sB + kQ * kLdC;             // [kP][kLdC]   chunk start state
  float* sX = sH + kP * kLdC;             // [kQ][kLdX]   raw x
  float* sM = sX + kQ * kLdX;             // [kQ][kLdM]
  float* s_dtv = sM + kQ * kLdM;
  float* s_cum = s_dtv + kQ;
  float* s_tmp = s_cum + kQ;
  const int c = blockIdx.x, hd = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int n = p.q_len[seq];
  if (c * kQ >= n) return;
  const int tok0 = p.q_start[seq] + c * kQ;
  const int valid = min(kQ, n - c * kQ);
  const int inner = p.H * kP, GN = p.G * kN, ld = inner + 2 * GN;
  const int grp = hd / (p.H / p.G);
  const float a_exp = __expf(p.A_log[hd]);
  chunk_gates(p, tok0, valid, hd, a_exp, s_dtv, s_cum, s_tmp);
  const float* hsrc = p.ws_state + (((size_t)seq * p.max_chunks + c) * p.H + hd) * (kP * kN);
  for (int i = tid; i < kQ * (kN / 4); i += 128) {
    const int j = i / (kN / 4), q4 = i - j * (kN / 4);
    float4 vb = make_float4(0.f, 0.f, 0.f, 0.f), vc = vb;
    if (j < valid) {
      const float* row = p.xbc + (size_t)(tok0 + j) * ld + inner + grp * kN + q4 * 4;
      vb = *reinterpret_cast<const float4*>(row);
      vc = *reinterpret_cast<const float4*>(row + GN);
    }
    *reinterpret_cast<float4*>(sB + j * kLdC + q4 * 4) = vb;
    *reinterpret_cast<float4*>(sC + j * kLdC + q4 * 4) = vc;
    *reinterpret_cast<float4*>(sH + j * kLdC + q4 * 4) = *reinterpret_cast<const float4*>(hsrc + j * kN + q4 * 4);
  }
  for (int i = tid; i < kQ * (kP / 4); i += 128) {
    const int j = i / (kP / 4), q4 = i - j * (kP / 4);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < valid) v = *reinterpret_cast<const float4*>(p.xbc + (size_t)(tok0 + j) * ld + hd * kP + q4 * 4);
    *reinterpret_cast<float4*>(sX + j * kLdX + q4 * 4) = v;
  }
  __syncthreads();
  const int g = lane >> 2, t = lane & 3;
  const int m0 = warp * 16;                                    // this warp's 16 tokens of the chunk
  // ---- G = C B^T for rows m0..m0+15, all 64 columns; K = 128
  float accg[kQ / 8][4];
#pragma unroll
  for (int nt = 0; nt < kQ / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) accg[nt][i] = 0.f;
  // ---- Y2 = C h_start^T for the same rows, 64 columns p; K = 128 (shares the A fragments)
  float acch[kP / 8][4];
#pragma unroll
  for (int nt = 0; nt < kP / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acch[nt][i] = 0.f;
#pragma unroll 2
  for (int k0 = 0; k0 < kN; k0 += 8) {
    const uint32_t a0 = to_tf32(sC[(m0 + g) * kLdC + k0 + t]);
    const uint32_t a1 = to_tf32(sC[(m0 + g + 8) * kLdC + k0 + t]);
    const uint32_t a2 = to_tf32(sC[(m0 + g) * kLdC + k0 + t + 4]);
    const uint32_t a3 = to_tf32(sC[(m0 + g + 8) * kLdC + k0 + t + 4]);
#pragma unroll
    for (int nt = 0; nt < kQ / 8; ++nt) {
      if (nt * 8 <= m0 + 15) {                                  // columns j beyond the warp's last row are masked anyway
        const uint32_t b0 = to_tf32(sB[(nt * 8 + g) * kLdC + k0 + t]);
        const uint32_t b1 = to_tf32(sB[(nt * 8 + g) * kLdC + k0 + t + 4]);
        mma_tf32(accg[nt], a0, a1, a2, a3, b0, b1);
      }
    }
#pragma unroll
    for (int nt = 0; nt < kP / 8; ++nt) {
      const uint32_t b0 = to_tf32(sH[(nt * 8 + g) * kLdC + k0 + t]);
      const uint32_t b1 = to_tf32(sH[(nt * 8 + g) * kLdC + k0 + t + 4]);
      mma_tf32(acch[nt], a0, a1, a2, a3, b0, b1);
    }
  }
  // ---- M_ij = G_ij exp(cum_i - cum_j) dtv_j for j <= i (0 above the diagonal), into shared memory
  {
    const int i0 = m0 + g, i1 = m0 + g + 8;
    const float ci0 = s_cum[i0], ci1 = s_cum[i1];
#pragma unroll
    for (int nt = 0; nt < kQ / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = nt * 8 + 2 * t + e;
        const float cj = s_cum[j], dj = s_dtv[j];
        sM[i0 * kLdM + j] = j <= i0 ? accg[nt][e] * __expf(ci0 - cj) * dj : 0.f;
        sM[i1 * kLdM + j] = j <= i1 ? accg[nt][2 + e] * __expf(ci1 - cj) * dj : 0.f;
      }
    }
  }
  __syncwarp();
  // ---- Y1 = M X for rows m0..m0+15, 64 columns p; K = tokens up to the warp's last row
  float accy[kP / 8][4];
#pragma unroll
  for (int nt = 0; nt < kP / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) accy[nt][i] = 0.f;
  for (int k0 = 0; k0 <= m0 + 15; k0 += 8) {
    const uint32_t a0 = to_tf32(sM[(m0 + g) * kLdM + k0 + t]);
    const uint32_t a1 = to_tf32(sM[(m0 + g + 8) * kLdM + k0 + t]);
    const uint32_t a2 = to_tf32(sM[(m0 + g) * kLdM + k0 + t + 4]);
    const uint32_t a3 = to_tf32(sM[(m0 + g + 8) * kLdM + k0 + t + 4]);
#pragma unroll
    for (int nt = 0; nt < kP / 8; ++nt) {
      const uint32_t b0 = to_tf32(sX[(k0 + t) * kLdX + nt * 8 + g]);
      const uint32_t b1 = to_tf32(sX[(k0 + t + 4) * kLdX + nt * 8 + g]);
      mma_tf32(accy[nt], a0, a1, a2, a3, b0, b1);
    }
  }
  // ---- y = Y1 + exp(cum_i) Y2 + D x
  const float dcoef = p.Dp[hd];
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    const int i = m0 + g + hr * 8;
    if (i >= valid) continue;
    const float ei = __expf(s_cum[i]);
    float* dst = p.out + (size_t)(tok0 + i) * inner + hd * kP;
#pragma unroll
    for (int nt = 0; nt < kP / 8; ++nt) {
      const int pc = nt * 8 + 2 * t;
      const float y0 = accy[nt][hr * 2] + ei * acch[nt][hr * 2] + dcoef * sX[i * kLdX + pc];
      const float y1 = accy[nt][hr * 2 + 1] + ei * acch[nt][hr * 2 + 1] + dcoef * sX[i * kLdX + pc + 1];
      *reinterpret_cast<float2*>(dst + pc) = make_float2(y0, y1);
    }
  }
}

constexpr size_t kSmemState = (size_t)(kQ * kLdX + kQ * kLdBn + 2 * kQ + 8) * sizeof(float);
constexpr size_t kSmemOut = (size_t)(3 * kQ * kLdC + kQ * kLdX + kQ * kLdM + 2 * kQ + 8) * sizeof(float);

}  // namespace

extern "C" {

// bytes of workspace for a batch of `num_seqs` sequences whose longest has `max_q_len` tokens
size_t mb_mamba2_ssd_ws_bytes(int num_seqs, int max_q_len, int H) {
  const size_t chunks = (size_t)((max_q_len + kQ - 1) / kQ);
  return (size_t)num_seqs * chunks * H * ((size_t)kP * kN + 1) * sizeof(float) + 256;
}

int mb_mamba2_ssd(const float* xbc, const void* dt, long long dt_ld, const float* A_log, const float* D,
                  const float* dt_bias, float* state, float* out, int H, int G, int P, int N,
                  const int* q_start, const int* q_len, const int* positions, const int* state_slots,
                  int num_seqs, int num_slots, int max_q_len, int write_state, void* ws, size_t ws_bytes,
                  uint32_t* status, cudaStream_t stream) {
  if (!xbc || !dt || !state || !out || !ws || num_seqs <= 0 || max_q_len <= 0 || H <= 0 || G <= 0 || H % G)
    return MB_ERR_BAD_ARG;
  if (P != kP || N != kN) return MB_ERR_UNSUPPORTED;
  if (ws_bytes < mb_mamba2_ssd_ws_bytes(num_seqs, max_q_len, H)) return MB_ERR_TOO_LARGE;
  if (((H * kP + 2 * G * kN) % 4) != 0) return MB_ERR_UNSUPPORTED;        // 16-byte row loads
  SsdParams p{};
  p.xbc = xbc; p.dt = reinterpret_cast<const __nv_bfloat16*>(dt); p.dt_ld = dt_ld;
  p.A_log = A_log; p.Dp = D; p.dt_bias = dt_bias; p.state = state; p.out = out;
  p.max_chunks = (max_q_len + kQ - 1) / kQ;
  p.ws_state = reinterpret_cast<float*>(ws);
  p.ws_decay = p.ws_state + (size_t)num_seqs * p.max_chunks * H * (kP * kN);
  p.q_start = q_start; p.q_len = q_len; p.positions = positions; p.state_slots = state_slots;
  p.H = H; p.G = G; p.num_slots = num_slots; p.write_state = write_state; p.status = status;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(ssd_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemState);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(ssd_chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemOut);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (p.max_chunks > 65535 || num_seqs > 65535) return MB_ERR_TOO_LARGE;
  const dim3 grid(p.max_chunks, H, num_seqs);
  cudaError_t e = mb::launch_kernel(ssd_chunk_state_kernel, grid, dim3(128), kSmemState, stream, p);
  if (e != cudaSuccess) return (int)e;
  e = mb::launch_kernel(ssd_state_scan_kernel, dim3(H, num_seqs), dim3(256), 0, stream, p);
  if (e != cudaSuccess) return (int)e;
  return (int)mb::launch_kernel(ssd_chunk_out_kernel, grid, dim3(128), kSmemOut, stream, p);
}

}  // extern "C"
