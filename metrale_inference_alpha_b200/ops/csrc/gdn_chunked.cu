// Chunked (parallel-in-time) prefill of the gated delta rule: a long prompt no longer walks its
// tokens one by one.
//
// Per value head, with unit-norm keys k_i, scaled unit-norm queries q_i, decay g_i in (0, 1] and
// write strength beta_i, the recurrence of the sequential kernel (recurrent.cu) is
//     d_i = beta_i (v_i - (g_i S_{i-1})^T k_i),   S_i = g_i S_{i-1} + k_i d_i^T,   o_i = S_i^T q_i.
// Inside a chunk of 64 tokens let G_i be the inclusive sum of log g and A the strictly lower
// triangular matrix A_ij = beta_i exp(G_i - G_j) (k_i . k_j). Unrolling the recurrence gives
//     (I + A) D = beta (.) V  -  (beta exp(G) (.) K) S_0            =>  D = U - W S_0
//     o_i = exp(G_i) q_i^T S_0 + sum_{j<=i} exp(G_i - G_j) (q_i . k_j) d_j
//     S_64 = exp(G_64) S_0 + sum_j exp(G_64 - G_j) k_j d_j^T
// where W and U solve the unit lower-triangular system for the two right-hand sides. Two launches
// for the whole ragged batch:
//   gdn_chunk_prep  per (chunk, head, sequence), everything that does not need the state: norms and
//                   gates, K K^T and Q K^T (64 x 64, K = 128; 3xTF32 split, so A is fp32-accurate),
//                   the forward substitution for W | U (one column per thread), and the decayed
//                   operands exp(G_i) q_i, exp(G_64 - G_j) k_j, the masked Q K^T.
//   gdn_chunk_scan  per (32-column slice of the state, head, sequence), the short recurrence over
//                   chunks with the state slice resident in shared memory: D = U - W S,
//                   o = (exp(G) Q) S + P D, S = exp(G_64) S + Kd^T D; four TF32 tensor-core
//                   products per chunk, operands prefetched with cp.async while the previous
//                   product runs.
// Products run as `mma.sync.m16n8k8` TF32 with fp32 accumulation: the operands are fp32
// activations and a 64-row chunk is below the 128-row tile at which tcgen05 pays for its TMEM
// round trip. The sequential kernel stays the oracle and serves decode / verify rows.
//
// Reference behaviour covered: kernels/gb10/common/gated_delta_rule_fla.cu (chunked WY form),
// gated_delta_rule.cu:8-16 (the recurrence), ssm_preprocess.cu (gates).
#include "common.cuh"

namespace {

constexpr int kC = 64;        // chunk length
constexpr int kD = 128;       // key dim = value dim
constexpr int kSlice = 32;    // value columns per scan CTA
// workspace record of one (sequence, chunk, value head), in floats
constexpr int kOffW = 0, kOffU = kC * kD, kOffKd = 2 * kC * kD, kOffQg = 3 * kC * kD, kOffP = 4 * kC * kD,
              kOffGam = kOffP + kC * kC, kRec = kOffGam + 64;

struct GdnParams {
  const float* conv;     // [T, 2 QK + V] fp32: q | k | v
  const float* ba;       // [T, 2 v_heads] fp32: b | a
  const float* A_log;
  const float* dt_bias;
  float* state;          // [slots, v_heads, kD, kD]
  float* out;            // [T, v_heads * kD]
  float* ws;
  const int* q_start;
  const int* q_len;
  const int* positions;
  const int* state_slots;
  int k_heads, v_heads, num_slots, max_chunks, write_state;
  uint32_t* status;
};

__device__ __forceinline__ uint32_t tf32(float f) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(f));
  return r;
}
__device__ __forceinline__ void mma8(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void split(float x, uint32_t& hi, uint32_t& lo) {
  hi = tf32(x);
  lo = tf32(x - __uint_as_float(hi));
}
__device__ __forceinline__ void cp16(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float* record(const GdnParams& p, int seq, int c, int vh) {
  return p.ws + (((size_t)seq * p.max_chunks + c) * p.v_heads + vh) * kRec;
}

// ------------------------------------------------------------------ per-chunk preparation
constexpr int kLdX = 2 * kD + 4;   // row [k (128) | q, later beta v (128)]; stride = 4 (mod 32): conflict-free row fragments
constexpr int kLdA = kC + 4;
constexpr size_t kSmemPrep = (size_t)(kC * kLdX + kC * kLdA + 3 * kC) * sizeof(float);

__global__ void __launch_bounds__(256) gdn_chunk_prep_kernel(const GdnParams p) {
  extern __shared__ __align__(16) float sm[];
  float* X = sm;
  float* A = X + kC * kLdX;
  float* sG = A + kC * kLdA;
  float* sBeta = sG + kC;
  float* sTmp = sBeta + kC;
  const int c = blockIdx.x, vh = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int n = p.q_len[seq];
  if (c * kC >= n) return;
  const int tok0 = p.q_start[seq] + c * kC;
  const int valid = min(kC, n - c * kC);
  const int kh = vh / (p.v_heads / p.k_heads);
  const int QK = p.k_heads * kD, V = p.v_heads * kD, ld = 2 * QK + V;
  float* rec = record(p, seq, c, vh);

  // unit-norm keys and scaled unit-norm queries, one warp per row
  for (int i = warp; i < kC; i += 8) {
    float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f), k4 = q4;
    if (i < valid) {
      const float* row = p.conv + (size_t)(tok0 + i) * ld;
      q4 = *reinterpret_cast<const float4*>(row + kh * kD + lane * 4);
      k4 = *reinterpret_cast<const float4*>(row + QK + kh * kD + lane * 4);
    }
    const float sq = mb::warp_sum(q4.x * q4.x + q4.y * q4.y + q4.z * q4.z + q4.w * q4.w);
    const float sk = mb::warp_sum(k4.x * k4.x + k4.y * k4.y + k4.z * k4.z + k4.w * k4.w);
    const float nq = rsqrtf(sq + 1e-6f) * rsqrtf((float)kD), nk = rsqrtf(sk + 1e-6f);
    *reinterpret_cast<float4*>(X + i * kLdX + lane * 4) = make_float4(k4.x * nk, k4.y * nk, k4.z * nk, k4.w * nk);
    *reinterpret_cast<float4*>(X + i * kLdX + kD + lane * 4) = make_float4(q4.x * nq, q4.y * nq, q4.z * nq, q4.w * nq);
  }
  // gates: log decay (inclusive prefix sum) and beta; rows past the end decay by 1 and write nothing
  if (tid < kC) {
    float lg = 0.f, beta = 0.f;
    if (tid < valid) {
      const float bb = p.ba[(size_t)(tok0 + tid) * 2 * p.v_heads + vh];
      const float aa = p.ba[(size_t)(tok0 + tid) * 2 * p.v_heads + p.v_heads + vh];
      const float sp = log1pf(__expf(fminf(aa + p.dt_bias[vh], 20.f)));
      lg = -__expf(fminf(p.A_log[vh], 20.f)) * sp;
      beta = 1.f / (1.f + __expf(-bb));
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, lg, o);
      if (lane >= o) lg += up;
    }
    sG[tid] = lg;
    sBeta[tid] = beta;
    if (tid == 31) sTmp[0] = lg;
  }
  __syncthreads();
  if (tid >= 32 && tid < kC) sG[tid] += sTmp[0];
  __syncthreads();

  // K K^T and Q K^T on the tensor cores (hi/lo split: three products each), lower triangle only
  {
    const int wr = (warp & 3) * 16, wc = (warp >> 2) * 32;
    float accK[4][4], accQ[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) accK[i][j] = accQ[i][j] = 0.f;
    for (int k0 = 0; k0 < kD; k0 += 8) {
      uint32_t akh[4], akl[4], aqh[4], aql[4];
      const float* r0 = X + (wr + g) * kLdX + k0 + t;
      const float* r1 = r0 + 8 * kLdX;
      split(r0[0], akh[0], akl[0]); split(r1[0], akh[1], akl[1]);
      split(r0[4], akh[2], akl[2]); split(r1[4], akh[3], akl[3]);
      split(r0[kD], aqh[0], aql[0]); split(r1[kD], aqh[1], aql[1]);
      split(r0[kD + 4], aqh[2], aql[2]); split(r1[kD + 4], aqh[3], aql[3]);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int n0 = wc + nt * 8;
        if (n0 > wr + 15) continue;                       // above the diagonal (same for the whole warp)
        const float* rb = X + (n0 + g) * kLdX + k0 + t;
        uint32_t b0h, b0l, b1h, b1l;
        split(rb[0], b0h, b0l);
        split(rb[4], b1h, b1l);
        mma8(accK[nt], akh, b0h, b1h); mma8(accK[nt], akl, b0h, b1h); mma8(accK[nt], akh, b0l, b1l);
        mma8(accQ[nt], aqh, b0h, b1h); mma8(accQ[nt], aql, b0h, b1h); mma8(accQ[nt], aqh, b0l, b1l);
      }
    }
    float* P = rec + kOffP;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int n0 = wc + nt * 8;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = wr + g + 8 * h;
        float pa[2], pp[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = n0 + 2 * t + e;
          const float dec = j <= i ? __expf(sG[i] - sG[j]) : 0.f;
          pa[e] = j < i ? sBeta[i] * dec * accK[nt][2 * h + e] : 0.f;
          pp[e] = dec * accQ[nt][2 * h + e];
        }
        *reinterpret_cast<float2*>(A + i * kLdA + n0 + 2 * t) = make_float2(pa[0], pa[1]);
        *reinterpret_cast<float2*>(P + i * kC + n0 + 2 * t) = make_float2(pp[0], pp[1]);
      }
    }
  }
  __syncthreads();
  // decayed operands of the scan, and the right-hand sides [beta exp(G) k | beta v] in place
  const float g_last = sG[kC - 1];
  for (int idx = tid; idx < kC * (kD / 4); idx += 256) {
    const int i = idx / (kD / 4), c4 = (idx % (kD / 4)) * 4;
    const float4 k4 = *reinterpret_cast<const float4*>(X + i * kLdX + c4);
    const float4 q4 = *reinterpret_cast<const float4*>(X + i * kLdX + kD + c4);
    const float gi = __expf(sG[i]), gl = i < valid ? __expf(g_last - sG[i]) : 0.f, bi = sBeta[i];
    *reinterpret_cast<float4*>(rec + kOffQg + i * kD + c4) = make_float4(q4.x * gi, q4.y * gi, q4.z * gi, q4.w * gi);
    *reinterpret_cast<float4*>(rec + kOffKd + i * kD + c4) = make_float4(k4.x * gl, k4.y * gl, k4.z * gl, k4.w * gl);
    const float w = bi * gi;
    *reinterpret_cast<float4*>(X + i * kLdX + c4) = make_float4(k4.x * w, k4.y * w, k4.z * w, k4.w * w);
    float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < valid) v4 = *reinterpret_cast<const float4*>(p.conv + (size_t)(tok0 + i) * ld + 2 * QK + vh * kD + c4);
    *reinterpret_cast<float4*>(X + i * kLdX + kD + c4) = make_float4(v4.x * bi, v4.y * bi, v4.z * bi, v4.w * bi);
  }
  if (tid == 0) rec[kOffGam] = __expf(g_last);
  __syncthreads();
  // forward substitution, one column of [W | U] per thread: x_i = b_i - sum_{j<i} A_ij x_j
  {
    const int col = tid;
    float* dst = rec + (col < kD ? kOffW + col : kOffU + col - kD);
    for (int i = 0; i < kC; ++i) {
      float acc = X[i * kLdX + col];
      if (i < valid) {
        const float* arow = A + i * kLdA;
        int j = 0;
        for (; j + 4 <= i; j += 4) {
          const float4 a4 = *reinterpret_cast<const float4*>(arow + j);
          acc -= a4.x * X[j * kLdX + col];
          acc -= a4.y * X[(j + 1) * kLdX + col];
          acc -= a4.z * X[(j + 2) * kLdX + col];
          acc -= a4.w * X[(j + 3) * kLdX + col];
        }
        for (; j < i; ++j) acc -= arow[j] * X[j * kLdX + col];
        X[i * kLdX + col] = acc;
      }
      dst[i * kD] = acc;
    }
  }
}

// ------------------------------------------------------------------ recurrence over chunks
constexpr int kLdW = kD + 4;        // A operands read by rows: stride = 4 (mod 32)
constexpr int kLdKd = kD + 8;       // A operand read transposed: stride = 8 (mod 32)
constexpr int kLdP = kC + 4;
constexpr int kLdS = kSlice + 8;    // B operands: stride = 8 (mod 32)
constexpr size_t kSmemScan =
    (size_t)(2 * kC * kLdW + kC * kLdKd + kC * kLdP + 2 * kC * kLdS + kD * kLdS) * sizeof(float);

__device__ __forceinline__ void load_tile(float* dst, int dst_ld, const float* src, int src_ld, int rows, int cols) {
  const int per_row = cols / 4;
  for (int idx = threadIdx.x; idx < rows * per_row; idx += 256) {
    const int r = idx / per_row, c4 = (idx - r * per_row) * 4;
    cp16(dst + r * dst_ld + c4, src + (size_t)r * src_ld + c4);
  }
}

__global__ void __launch_bounds__(256) gdn_chunk_scan_kernel(const GdnParams p) {
  extern __shared__ __align__(16) float sm[];
  float* sW = sm;                          // [kC][kLdW]
  float* sQ = sW + kC * kLdW;              // [kC][kLdW]   exp(G) q
  float* sKd = sQ + kC * kLdW;             // [kC][kLdKd]  exp(G_64 - G) k
  float* sP = sKd + kC * kLdKd;            // [kC][kLdP]
  float* sU = sP + kC * kLdP;              // [kC][kLdS]
  float* sV = sU + kC * kLdS;              // [kC][kLdS]   D = U - W S
  float* sS = sV + kC * kLdS;              // [kD][kLdS]   the state slice
  const int slice = blockIdx.x, vh = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int n = p.q_len[seq];
  if (n <= 0) return;
  const int q0 = p.q_start[seq];
  const int slot = p.state_slots[seq];
  if (slot < 0 || slot >= p.num_slots) {
    if (p.status && tid == 0) atomicCAS(p.status, 0u, MB_ST_BOUNDS);
    return;
  }
  const int V = p.v_heads * kD;
  const int chunks = (n + kC - 1) / kC;
  float* hs = p.state + (((size_t)slot * p.v_heads + vh) * kD) * kD + slice * kSlice;
  const bool fresh = p.positions[q0] == 0;
  for (int idx = tid; idx < kD * (kSlice / 4); idx += 256) {
    const int k = idx / (kSlice / 4), c4 = (idx % (kSlice / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!fresh) v = *reinterpret_cast<const float4*>(hs + (size_t)k * kD + c4);
    *reinterpret_cast<float4*>(sS + k * kLdS + c4) = v;
  }
  auto issue_wu = [&](int c) {
    if (c < chunks) {
      const float* rec = record(p, seq, c, vh);
      load_tile(sW, kLdW, rec + kOffW, kD, kC, kD);
      load_tile(sU, kLdS, rec + kOffU + slice * kSlice, kD, kC, kSlice);
    }
    cp_commit();
  };
  auto issue_qp = [&](int c) {
    if (c < chunks) {
      const float* rec = record(p, seq, c, vh);
      load_tile(sQ, kLdW, rec + kOffQg, kD, kC, kD);
      load_tile(sP, kLdP, rec + kOffP, kC, kC, kC);
    }
    cp_commit();
  };
  auto issue_kd = [&](int c) {
    if (c < chunks) load_tile(sKd, kLdKd, record(p, seq, c, vh) + kOffKd, kD, kC, kD);
    cp_commit();
  };
  issue_wu(0);
  issue_qp(0);
  issue_kd(0);
  const int wr = (warp & 3) * 16, wc = (warp >> 2) * 16;     // 64 x 32 products: 16 x 16 per warp
  for (int c = 0; c < chunks; ++c) {
    const int valid = min(kC, n - c * kC);
    const float gam = record(p, seq, c, vh)[kOffGam];
    // ---- D = U - W S
    cp_wait<2>();
    __syncthreads();
    {
      float acc[2][4] = {};
      for (int k0 = 0; k0 < kD; k0 += 8) {
        uint32_t a[4];
        const float* r0 = sW + (wr + g) * kLdW + k0 + t;
        a[0] = tf32(r0[0]); a[1] = tf32(r0[8 * kLdW]); a[2] = tf32(r0[4]); a[3] = tf32(r0[8 * kLdW + 4]);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const float* b = sS + (k0 + t) * kLdS + wc + nt * 8 + g;
          mma8(acc[nt], a, tf32(b[0]), tf32(b[4 * kLdS]));
        }
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int o = (wr + g + 8 * h) * kLdS + wc + nt * 8 + 2 * t;
          const float2 u = *reinterpret_cast<const float2*>(sU + o);
          *reinterpret_cast<float2*>(sV + o) = make_float2(u.x - acc[nt][2 * h], u.y - acc[nt][2 * h + 1]);
        }
    }
    __syncthreads();
    issue_wu(c + 1);
    // ---- o = (exp(G) Q) S + P D
    cp_wait<2>();
    __syncthreads();
    {
      float acc[2][4] = {};
      for (int k0 = 0; k0 < kD; k0 += 8) {
        uint32_t a[4];
        const float* r0 = sQ + (wr + g) * kLdW + k0 + t;
        a[0] = tf32(r0[0]); a[1] = tf32(r0[8 * kLdW]); a[2] = tf32(r0[4]); a[3] = tf32(r0[8 * kLdW + 4]);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const float* b = sS + (k0 + t) * kLdS + wc + nt * 8 + g;
          mma8(acc[nt], a, tf32(b[0]), tf32(b[4 * kLdS]));
        }
      }
      for (int k0 = 0; k0 <= wr + 8; k0 += 8) {            // P is lower triangular
        uint32_t a[4];
        const float* r0 = sP + (wr + g) * kLdP + k0 + t;
        a[0] = tf32(r0[0]); a[1] = tf32(r0[8 * kLdP]); a[2] = tf32(r0[4]); a[3] = tf32(r0[8 * kLdP + 4]);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const float* b = sV + (k0 + t) * kLdS + wc + nt * 8 + g;
          mma8(acc[nt], a, tf32(b[0]), tf32(b[4 * kLdS]));
        }
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int i = wr + g + 8 * h;
          if (i < valid)
            *reinterpret_cast<float2*>(p.out + (size_t)(q0 + c * kC + i) * V + vh * kD + slice * kSlice + wc + nt * 8 + 2 * t) =
                make_float2(acc[nt][2 * h], acc[nt][2 * h + 1]);
        }
    }
    __syncthreads();
    issue_qp(c + 1);
    // ---- S = exp(G_64) S + Kd^T D   (128 x 32, K = 64): 16 state rows per warp
    cp_wait<2>();
    __syncthreads();
    {
      const int m0 = warp * 16;
      float acc[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float2 s = *reinterpret_cast<const float2*>(sS + (m0 + g + 8 * h) * kLdS + nt * 8 + 2 * t);
          acc[nt][2 * h] = gam * s.x;
          acc[nt][2 * h + 1] = gam * s.y;
        }
      for (int k0 = 0; k0 < kC; k0 += 8) {
        uint32_t a[4];
        const float* r0 = sKd + (k0 + t) * kLdKd + m0 + g;
        a[0] = tf32(r0[0]); a[1] = tf32(r0[8]); a[2] = tf32(r0[4 * kLdKd]); a[3] = tf32(r0[4 * kLdKd + 8]);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const float* b = sV + (k0 + t) * kLdS + nt * 8 + g;
          mma8(acc[nt], a, tf32(b[0]), tf32(b[4 * kLdS]));
        }
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          *reinterpret_cast<float2*>(sS + (m0 + g + 8 * h) * kLdS + nt * 8 + 2 * t) =
              make_float2(acc[nt][2 * h], acc[nt][2 * h + 1]);
    }
    __syncthreads();
    issue_kd(c + 1);
  }
  cp_wait<0>();
  if (p.write_state) {
    for (int idx = tid; idx < kD * (kSlice / 4); idx += 256) {
      const int k = idx / (kSlice / 4), c4 = (idx % (kSlice / 4)) * 4;
      *reinterpret_cast<float4*>(hs + (size_t)k * kD + c4) = *reinterpret_cast<const float4*>(sS + k * kLdS + c4);
    }
  }
}

}  // namespace

extern "C" {

size_t mb_gdn_chunked_ws_bytes(int num_seqs, int max_q_len, int v_heads) {
  const size_t chunks = (size_t)((max_q_len + kC - 1) / kC);
  return (size_t)num_seqs * chunks * v_heads * kRec * sizeof(float);
}

// Chunked gated delta rule over a ragged batch (key dim = value dim = 128). Same arguments and
// results as mb_gdn_recurrence plus the workspace. Returns 0, a negative MB_ERR_* or a CUDA error.
int mb_gdn_chunked(const float* conv, const float* ba, const float* A_log, const float* dt_bias, float* state,
                   float* out, int k_heads, int v_heads, int k_dim, int v_dim, const int* q_start, const int* q_len,
                   const int* positions, const int* state_slots, int num_seqs, int num_slots, int max_q_len,
                   int write_state, void* ws, size_t ws_bytes, uint32_t* status, cudaStream_t stream) {
  if (k_dim != kD || v_dim != kD || v_heads % k_heads != 0 || num_seqs <= 0 || max_q_len <= 0) return MB_ERR_BAD_ARG;
  if (ws_bytes < mb_gdn_chunked_ws_bytes(num_seqs, max_q_len, v_heads)) return MB_ERR_BAD_ARG;
  GdnParams p;
  p.conv = conv; p.ba = ba; p.A_log = A_log; p.dt_bias = dt_bias; p.state = state; p.out = out;
  p.ws = reinterpret_cast<float*>(ws);
  p.q_start = q_start; p.q_len = q_len; p.positions = positions; p.state_slots = state_slots;
  p.k_heads = k_heads; p.v_heads = v_heads; p.num_slots = num_slots;
  p.max_chunks = (max_q_len + kC - 1) / kC;
  p.write_state = write_state; p.status = status;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemPrep);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemScan);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (p.max_chunks > 65535 || num_seqs > 65535 || v_heads > 65535) return MB_ERR_TOO_LARGE;
  cudaError_t e = mb::launch_kernel(gdn_chunk_prep_kernel, dim3(p.max_chunks, v_heads, num_seqs), dim3(256), kSmemPrep, stream, p);
  if (e != cudaSuccess) return (int)e;
  return (int)mb::launch_kernel(gdn_chunk_scan_kernel, dim3(kD / kSlice, v_heads, num_seqs), dim3(256), kSmemScan, stream, p);
}

}  // extern "C"
