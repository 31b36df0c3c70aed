// Chunked prefill of Kimi delta attention (the per-channel gated delta rule of kda.cu) for long rows.
//
// Over a chunk of C = 32 positions of one head (i the query row, j the key column, d a channel, S the state
// [k][v], gc the inclusive cumulative log-decay inside the chunk):
//   A[i,j]     = -beta[i] sum_d k[i,d] k[j,d] exp(gc[i,d] - gc[j,d])        j < i
//   A          <- (I - A)^-1 by forward substitution (row i += row i @ rows < i), unit diagonal
//   u = A (beta v)            w = A (beta k exp(gc))          v_new = u - w S
//   out[i]     = (scale q[i] exp(gc[i])) S + sum_{j<=i} intra[i,j] v_new[j],
//                intra[i,j] = scale sum_d q[i,d] k[j,d] exp(gc[i,d] - gc[j,d])
//   S          <- exp(gc[C-1]) (.) S + (k exp(gc[C-1] - gc))^T v_new
// Every exponent is <= 0, so nothing overflows however strong the decay.
//
// Two kernels. `prep` works on every (sequence, chunk, head) independently: l2 norms, gate law, beta,
// cumulative decay, A with its inverse, u, w, the decayed q and k and the intra-chunk matrix go to a
// workspace. `scan` walks the chunks of a sequence in order with the state resident in shared memory; the
// value dimension is split over four CTAs per head (state columns are independent), so one long prompt
// keeps 4 x heads CTAs busy instead of `heads`, and inside a chunk everything is small dense products
// with no per-token dependency. Rows past the end of a sequence enter as k = v = beta = gate = 0, which
// leaves A, the state and the real rows untouched. The sigmoid-gated output norm needs a whole head and
// runs as a third, row-parallel kernel.
//
// The token-by-token kernel stays the path for decode and verify rows; the fp32 restatement
// ops/reference.py::kda_chunk states this algorithm and is checked against the token recurrence.
// Reference behaviour covered: kernels/gb10/common/kda_chunk.cu (kda_chunk_prepare, kda_chunk_scan).
#include "common.cuh"

namespace {

constexpr int kC = 32;            // chunk length
constexpr int kD = 128;           // head dim (key and value)
constexpr int kLd = kD + 1;       // padded row: rows i and j fall on different banks for the same channel
constexpr int kVs = 4;            // value-dimension splits of the scan
constexpr int kCols = kD / kVs;   // 32 state columns per scan CTA
constexpr int kScanThreads = 512, kWarps = kScanThreads / 32, kRw = kC / kWarps, kSr = kD / kWarps;   // rows per warp: chunk, state
// one stage of the scan's operands in shared memory, in floats
constexpr int kStW = 0, kStQg = kC * kD, kStKd = 2 * kC * kD, kStU = 3 * kC * kD, kStIn = kStU + kC * kCols,
              kStGl = kStIn + kC * kC, kStage = kStGl + kD;
// workspace per (sequence, chunk, head), in floats
constexpr int kOffU = 0, kOffW = kC * kD, kOffQg = 2 * kC * kD, kOffKd = 3 * kC * kD, kOffIntra = 4 * kC * kD,
              kOffGlast = 4 * kC * kD + kC * kC, kWsStride = 4 * kC * kD + kC * kC + kD;

__device__ __forceinline__ void cp16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(mb::smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct Seqs {
  const int* q_start;
  const int* q_len;
  const int* positions;
  const int* state_slots;
  int num_slots;
};

struct PrepArgs {
  const float* conv;      // [T, 3 H D]
  const float* g_raw;     // [T, H D]
  const float* b_raw;     // [T, b_ld]
  int b_ld;
  const float* A_log;     // [H]
  const float* dt_bias;   // [H D]
  float lower_bound;
  int H, max_chunks;
  Seqs sm;
  float* ws;
};

__global__ void __launch_bounds__(256) kda_chunk_prep_kernel(const PrepArgs a) {
  extern __shared__ __align__(16) float smem[];
  float* kn = smem;                       // [C][kLd]  l2-normalised k, later beta k exp(gc)
  float* qn = kn + kC * kLd;              // [C][kLd]  scale * l2-normalised q
  float* vb = qn + kC * kLd;              // [C][kLd]  beta v
  float* gc = vb + kC * kLd;              // [C][kLd]  gate, then its inclusive cumulative sum
  float* A = gc + kC * kLd;               // [C][C + 1]
  float* beta = A + kC * (kC + 1);        // [C]
  const int c = blockIdx.x, hd = blockIdx.y, seq = blockIdx.z;
  const int n = a.sm.q_len[seq];
  if (c * kC >= n) return;
  const int q0 = a.sm.q_start[seq] + c * kC;
  const int rows = min(kC, n - c * kC);
  const int HD = a.H * kD;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float a_exp = __expf(fminf(a.A_log[hd], 20.f));
  const float scale = rsqrtf((float)kD);
  // 1. rows: l2 norms, gate law, beta
  for (int i = warp; i < kC; i += 8) {
    float q4[4], k4[4], v4[4], g4[4];
    float bt = 0.f;
    if (i < rows) {
      const size_t row = (size_t)(q0 + i);
      const float* cr = a.conv + row * 3 * HD + hd * kD;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int d = lane + 32 * e;
        q4[e] = cr[d];
        k4[e] = cr[HD + d];
        v4[e] = cr[2 * HD + d];
        g4[e] = a.lower_bound / (1.f + __expf(-a_exp * (a.g_raw[row * HD + hd * kD + d] + a.dt_bias[hd * kD + d])));
      }
      bt = 1.f / (1.f + __expf(-a.b_raw[row * a.b_ld + hd]));
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) q4[e] = k4[e] = v4[e] = g4[e] = 0.f;
    }
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      sq = fmaf(q4[e], q4[e], sq);
      sk = fmaf(k4[e], k4[e], sk);
    }
    sq = mb::warp_sum(sq);
    sk = mb::warp_sum(sk);
    const float nq = rsqrtf(sq + 1e-6f) * scale, nk = rsqrtf(sk + 1e-6f);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int d = lane + 32 * e;
      kn[i * kLd + d] = i < rows ? k4[e] * nk : 0.f;
      qn[i * kLd + d] = i < rows ? q4[e] * nq : 0.f;
      vb[i * kLd + d] = v4[e] * bt;
      gc[i * kLd + d] = g4[e];
    }
    if (lane == 0) beta[i] = bt;
  }
  __syncthreads();
  // 2. inclusive cumulative decay per channel
  if (threadIdx.x < kD) {
    float acc = 0.f;
    for (int i = 0; i < kC; ++i) {
      acc += gc[i * kLd + threadIdx.x];
      gc[i * kLd + threadIdx.x] = acc;
    }
  }
  __syncthreads();
  float* wsb = a.ws + ((size_t)((size_t)seq * a.max_chunks + c) * a.H + hd) * kWsStride;
  // 3. A (strictly lower) and the intra-chunk matrix (lower incl. diagonal)
  for (int p = threadIdx.x; p < kC * kC; p += 256) {
    const int i = p / kC, j = p - i * kC;
    float sa = 0.f, sb = 0.f;
    if (j <= i) {
      for (int d = 0; d < kD; ++d) {
        const float e = __expf(gc[i * kLd + d] - gc[j * kLd + d]);
        const float kj = kn[j * kLd + d] * e;
        sa = fmaf(kn[i * kLd + d], kj, sa);
        sb = fmaf(qn[i * kLd + d], kj, sb);
      }
    }
    A[i * (kC + 1) + j] = j < i ? -beta[i] * sa : 0.f;
    wsb[kOffIntra + p] = j <= i ? sb : 0.f;
  }
  // decayed q and k for the scan, and the chunk's total decay (reads kn before step 5 rescales it)
  for (int p = threadIdx.x; p < kC * kD; p += 256) {
    const int i = p / kD, d = p - i * kD;
    const float g = gc[i * kLd + d], gl = gc[(kC - 1) * kLd + d];
    wsb[kOffQg + p] = qn[i * kLd + d] * __expf(g);
    wsb[kOffKd + p] = kn[i * kLd + d] * __expf(gl - g);
  }
  if (threadIdx.x < kD) wsb[kOffGlast + threadIdx.x] = gc[(kC - 1) * kLd + threadIdx.x];
  __syncthreads();
  // 4. (I - A)^-1 by forward substitution; one warp, lane = column
  if (warp == 0) {
    for (int i = 1; i < kC; ++i) {
      float acc = A[i * (kC + 1) + lane];
      for (int j = 0; j < i; ++j) acc = fmaf(A[i * (kC + 1) + j], A[j * (kC + 1) + lane], acc);
      __syncwarp();
      if (lane < i) A[i * (kC + 1) + lane] = acc;
      __syncwarp();
    }
    A[lane * (kC + 1) + lane] = 1.f;
  }
  // 5. kn <- beta k exp(gc)
  for (int p = threadIdx.x; p < kC * kD; p += 256) {
    const int i = p / kD, d = p - i * kD;
    kn[i * kLd + d] *= beta[i] * __expf(gc[i * kLd + d]);
  }
  __syncthreads();
  // 6. u = A vb, w = A kn
  {
    const int d = threadIdx.x & (kD - 1), i0 = (threadIdx.x >> 7) * (kC / 2);
    for (int i = i0; i < i0 + kC / 2; ++i) {
      float su = 0.f, sw = 0.f;
      for (int j = 0; j <= i; ++j) {
        const float aij = A[i * (kC + 1) + j];
        su = fmaf(aij, vb[j * kLd + d], su);
        sw = fmaf(aij, kn[j * kLd + d], sw);
      }
      wsb[kOffU + i * kD + d] = su;
      wsb[kOffW + i * kD + d] = sw;
    }
  }
}

struct ScanArgs {
  const float* ws;
  float* state;     // [slots, H, D, D]
  float* out;       // [T, H D]
  int H, max_chunks;
  Seqs sm;
  int write_state;
  uint32_t* status;
};

// grid (H * kVs, sequences); 512 threads (one CTA per SM: four warps per scheduler hide the shared-memory
// latency of the small products): warp r owns output rows r and r + 16 of the chunk and state rows
// [8 r, 8 r + 8); lane = state column
__global__ void __launch_bounds__(kScanThreads) kda_chunk_scan_kernel(const ScanArgs a) {
  extern __shared__ __align__(16) float smem[];
  float* S = smem;                      // [D][kCols]
  float* stage0 = S + kD * kCols;       // two stages of a chunk's operands: the next chunk streams in (cp.async)
                                        // while the current one is computed
  const int hd = blockIdx.x / kVs, vs = blockIdx.x - hd * kVs, seq = blockIdx.y;
  const int n = a.sm.q_len[seq];
  if (n <= 0) return;
  const int slot = a.sm.state_slots[seq];
  if (slot < 0 || slot >= a.sm.num_slots) {
    if (a.status && threadIdx.x == 0) atomicCAS(a.status, 0u, MB_ST_BOUNDS);
    return;
  }
  const int q0 = a.sm.q_start[seq];
  const int col = threadIdx.x & 31, r = threadIdx.x >> 5;
  const int HD = a.H * kD;
  float* st = a.state + (((size_t)slot * a.H + hd) * kD) * kD + vs * kCols + col;
  const bool fresh = a.sm.positions[q0] == 0;
  for (int k = r * kSr; k < r * kSr + kSr; ++k) S[k * kCols + col] = fresh ? 0.f : st[(size_t)k * kD];
  const int nchunks = (n + kC - 1) / kC;
  float* vn_s = stage0 + 2 * kStage;    // [C][kCols]
  auto issue = [&](int c) {
    const float* wsb = a.ws + ((size_t)((size_t)seq * a.max_chunks + c) * a.H + hd) * kWsStride;
    float* st_ = stage0 + (c & 1) * kStage;
    for (int p = threadIdx.x; p < kC * kD / 4; p += kScanThreads) {
      cp16(st_ + kStW + 4 * p, wsb + kOffW + 4 * p);
      cp16(st_ + kStQg + 4 * p, wsb + kOffQg + 4 * p);
      cp16(st_ + kStKd + 4 * p, wsb + kOffKd + 4 * p);
    }
    for (int p = threadIdx.x; p < kC * kCols / 4; p += kScanThreads) {
      const int i = p >> 3, q4 = p & 7;
      cp16(st_ + kStU + i * kCols + 4 * q4, wsb + kOffU + i * kD + vs * kCols + 4 * q4);
    }
    for (int p = threadIdx.x; p < kC * kC / 4; p += kScanThreads) cp16(st_ + kStIn + 4 * p, wsb + kOffIntra + 4 * p);
    if (threadIdx.x < kD / 4) cp16(st_ + kStGl + 4 * threadIdx.x, wsb + kOffGlast + 4 * threadIdx.x);
    cp_commit();
  };
  issue(0);
  for (int c = 0; c < nchunks; ++c) {
    __syncthreads();                                    // everyone is done with the stage the next chunk lands in
    if (c + 1 < nchunks) {
      issue(c + 1);
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();                                    // this chunk's operands (all threads' copies) are visible
    const float* st_ = stage0 + (c & 1) * kStage;
    const float *w_s = st_ + kStW, *qg_s = st_ + kStQg, *kd_s = st_ + kStKd, *u_s = st_ + kStU, *in_s = st_ + kStIn,
                *gl_s = st_ + kStGl;
    // v_new = u - w S, and the part of the output that reads the old state: four state rows per step, the
    // w / q operands as 16-byte broadcast reads shared by the chunk rows this warp owns
    float o[kRw], sv[kRw];
#pragma unroll
    for (int e = 0; e < kRw; ++e) o[e] = sv[e] = 0.f;
#pragma unroll 2
    for (int k = 0; k < kD; k += 4) {
      const float s0 = S[k * kCols + col], s1 = S[(k + 1) * kCols + col], s2 = S[(k + 2) * kCols + col],
                  s3 = S[(k + 3) * kCols + col];
#pragma unroll
      for (int e = 0; e < kRw; ++e) {
        const int i = r + kWarps * e;
        const float4 w4 = *reinterpret_cast<const float4*>(&w_s[i * kD + k]);
        const float4 q4 = *reinterpret_cast<const float4*>(&qg_s[i * kD + k]);
        sv[e] = fmaf(w4.x, s0, sv[e]);
        sv[e] = fmaf(w4.y, s1, sv[e]);
        sv[e] = fmaf(w4.z, s2, sv[e]);
        sv[e] = fmaf(w4.w, s3, sv[e]);
        o[e] = fmaf(q4.x, s0, o[e]);
        o[e] = fmaf(q4.y, s1, o[e]);
        o[e] = fmaf(q4.z, s2, o[e]);
        o[e] = fmaf(q4.w, s3, o[e]);
      }
    }
#pragma unroll
    for (int e = 0; e < kRw; ++e) {
      const int i = r + kWarps * e;
      vn_s[i * kCols + col] = u_s[i * kCols + col] - sv[e];
    }
    __syncthreads();
    const int rows = min(kC, n - c * kC);
#pragma unroll
    for (int e = 0; e < kRw; ++e) {
      const int i = r + kWarps * e;
      float so = o[e];
      for (int j = 0; j <= i; ++j) so = fmaf(in_s[i * kC + j], vn_s[j * kCols + col], so);
      if (i < rows) a.out[(size_t)(q0 + c * kC + i) * HD + hd * kD + vs * kCols + col] = so;
    }
    // S <- exp(gc_last) S + kd^T v_new: this thread's column of v_new in registers, kd as 16-byte broadcast reads
    {
      float vn[kC];
#pragma unroll
      for (int i = 0; i < kC; ++i) vn[i] = vn_s[i * kCols + col];
      for (int k = r * kSr; k < r * kSr + kSr; k += 4) {
        float s0 = S[k * kCols + col] * __expf(gl_s[k]), s1 = S[(k + 1) * kCols + col] * __expf(gl_s[k + 1]),
              s2 = S[(k + 2) * kCols + col] * __expf(gl_s[k + 2]), s3 = S[(k + 3) * kCols + col] * __expf(gl_s[k + 3]);
#pragma unroll
        for (int i = 0; i < kC; ++i) {
          const float4 k4 = *reinterpret_cast<const float4*>(&kd_s[i * kD + k]);
          s0 = fmaf(k4.x, vn[i], s0);
          s1 = fmaf(k4.y, vn[i], s1);
          s2 = fmaf(k4.z, vn[i], s2);
          s3 = fmaf(k4.w, vn[i], s3);
        }
        S[k * kCols + col] = s0;
        S[(k + 1) * kCols + col] = s1;
        S[(k + 2) * kCols + col] = s2;
        S[(k + 3) * kCols + col] = s3;
      }
    }
  }
  if (a.write_state)
    for (int k = r * kSr; k < r * kSr + kSr; ++k) st[(size_t)k * kD] = S[k * kCols + col];
}

// y = o * rsqrt(mean(o^2) + eps) * w * sigmoid(gate), one CTA per (row, head)
__global__ void __launch_bounds__(kD)
kda_out_norm_kernel(const float* __restrict__ o, const __nv_bfloat16* __restrict__ gate, long long gate_ld,
                    const float* __restrict__ w, __nv_bfloat16* __restrict__ y, int H, float eps) {
  __shared__ float red[kD / 32];
  const size_t row = blockIdx.x;
  const int hd = blockIdx.y, v = threadIdx.x;
  const float x = o[row * H * kD + hd * kD + v];
  const float s = mb::warp_sum(x * x);
  if ((v & 31) == 0) red[v >> 5] = s;
  __syncthreads();
  const float tot = red[0] + red[1] + red[2] + red[3];
  const float g = __bfloat162float(gate[row * gate_ld + hd * kD + v]);
  y[row * H * kD + hd * kD + v] = __float2bfloat16(x * rsqrtf(tot / kD + eps) * w[v] / (1.f + __expf(-g)));
}

}  // namespace

extern "C" size_t mb_kda_chunked_ws_bytes(int num_seqs, int max_q_len, int H) {
  const size_t chunks = (size_t)((max_q_len + kC - 1) / kC);
  return (size_t)num_seqs * chunks * H * kWsStride * sizeof(float);
}

struct MbKdaChunkedArgs {
  const void* conv;
  const void* g_raw;
  const void* b_raw;
  int b_ld;
  const void* A_log;
  const void* dt_bias;
  float lower_bound;
  void* state;
  void* out;          // fp32 [T, H D]
  void* out_norm;     // bf16 [T, H D] or null
  const void* out_gate;
  long long gate_ld;
  const void* norm_w;
  float eps;
  int H, D;
  const void* q_start;
  const void* q_len;
  const void* positions;
  const void* state_slots;
  int num_seqs, num_slots, max_q_len, total_rows, write_state;
  void* ws;
  size_t ws_bytes;
  void* status;
};

extern "C" int mb_kda_chunked(const MbKdaChunkedArgs* p, cudaStream_t stream) {
  if (!p || !p->conv || !p->g_raw || !p->b_raw || !p->state || !p->out || !p->ws || p->num_seqs <= 0 || p->H <= 0 ||
      p->max_q_len <= 0)
    return MB_ERR_BAD_ARG;
  if (p->D != kD) return MB_ERR_UNSUPPORTED;
  if (p->out_norm && (!p->norm_w || !p->out_gate)) return MB_ERR_BAD_ARG;
  if (p->ws_bytes < mb_kda_chunked_ws_bytes(p->num_seqs, p->max_q_len, p->H)) return MB_ERR_TOO_LARGE;
  const int max_chunks = (p->max_q_len + kC - 1) / kC;
  const Seqs sm{static_cast<const int*>(p->q_start), static_cast<const int*>(p->q_len),
                static_cast<const int*>(p->positions), static_cast<const int*>(p->state_slots), p->num_slots};
  PrepArgs pa{static_cast<const float*>(p->conv), static_cast<const float*>(p->g_raw), static_cast<const float*>(p->b_raw),
              p->b_ld, static_cast<const float*>(p->A_log), static_cast<const float*>(p->dt_bias), p->lower_bound, p->H,
              max_chunks, sm, static_cast<float*>(p->ws)};
  const size_t prep_smem = (size_t)(4 * kC * kLd + kC * (kC + 1) + kC) * sizeof(float);
  const size_t scan_smem = (size_t)(kD * kCols + 2 * kStage + kC * kCols) * sizeof(float);
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(kda_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prep_smem);
    cudaFuncSetAttribute(kda_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)scan_smem);
    attr = true;
  }
  kda_chunk_prep_kernel<<<dim3(max_chunks, p->H, p->num_seqs), 256, prep_smem, stream>>>(pa);
  ScanArgs sa{static_cast<const float*>(p->ws), static_cast<float*>(p->state), static_cast<float*>(p->out), p->H, max_chunks,
              sm, p->write_state, static_cast<uint32_t*>(p->status)};
  kda_chunk_scan_kernel<<<dim3(p->H * kVs, p->num_seqs), kScanThreads, scan_smem, stream>>>(sa);
  if (p->out_norm && p->total_rows > 0)
    kda_out_norm_kernel<<<dim3(p->total_rows, p->H), kD, 0, stream>>>(
        static_cast<const float*>(p->out), static_cast<const __nv_bfloat16*>(p->out_gate), p->gate_ld,
        static_cast<const float*>(p->norm_w), static_cast<__nv_bfloat16*>(p->out_norm), p->H, p->eps);
  return (int)cudaGetLastError();
}
