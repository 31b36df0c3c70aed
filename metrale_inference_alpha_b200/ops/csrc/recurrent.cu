// Recurrent-state kernels over a ragged batch (decode rows, verify rows and prefill chunks in
// one launch): causal conv1d with a carried window, the gated-delta-net recurrence and the
// Mamba2 selective scan. State lives in fp32 pools indexed by a per-sequence slot id; a
// sequence whose first row is at position 0 starts from a zero state.
//
//   mb_causal_conv1d   y[t, c] = act(bias[c] + sum_k win[k] * w[c, k]); one thread per channel
//                      walks its sequence's tokens with the window in registers.
//   mb_gdn_recurrence  per (value head, sequence): q/k l2-norm, decay/beta gates, then
//                      v' = (v - g (h^T k)) beta; h = g h + k (x) v'; o = h^T q / sqrt(dk).
//                      Thread v owns column h[:, v] in registers.
//   mb_mamba2_scan     per (head, sequence): dt = softplus(dt + bias); dA = exp(-exp(A_log) dt);
//                      h = dA h + dt x (x) B; y = h C + D x. Two threads own one row h[p, :].
//
// Speculative verification: with `write_state` = 0 a kernel computes its outputs from the stored
// state and leaves the state untouched; once the number of accepted tokens is known the same
// kernel is run again over the retained inputs with q_len = accepted count and `write_out` = 0,
// which advances the state by exactly the accepted tokens with bit-identical arithmetic
// (write-on-accept; role of kernels/gb10/common/gated_delta_rule_wy4_woa.cu and
// gated_delta_rule_carry.cu, crates/model-engine/src/model/gdn_carry.rs).
//
// Reference behaviour covered: kernels/gb10/common/causal_conv1d.cu (update / fwd / prefill
// state), ssm_preprocess.cu (compute_gdn_gates), gated_delta_rule.cu (decode_f32_strided and
// the persistent prefill variants), mamba2_ssm_decode.cu (decode / prefill).
#include "common.cuh"

namespace {

struct SeqMeta {
  const int* q_start;
  const int* q_len;
  const int* positions;
  const int* state_slots;
  int num_slots;
};

// ------------------------------------------------------------------ conv1d
template <int TAPS>
__global__ void __launch_bounds__(128)
conv1d_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, int C, const float* __restrict__ w,
              const float* __restrict__ bias, float* __restrict__ state, float* __restrict__ out,
              SeqMeta sm, int activation, int write_state, int write_out, uint32_t* status) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int seq = blockIdx.y;
  if (c >= C) return;
  const int n = sm.q_len[seq];
  if (n <= 0) return;
  const int q0 = sm.q_start[seq];
  const int slot = sm.state_slots[seq];
  if (slot < 0 || slot >= sm.num_slots) {
    if (status) atomicCAS(status, 0u, MB_ST_BOUNDS);
    return;
  }
  float win[TAPS];
  float wk[TAPS];
#pragma unroll
  for (int k = 0; k < TAPS; ++k) wk[k] = w[(size_t)c * TAPS + k];
  float* st = state + ((size_t)slot * C + c) * (TAPS - 1);
  const bool fresh = sm.positions[q0] == 0;
#pragma unroll
  for (int k = 0; k < TAPS - 1; ++k) win[k] = fresh ? 0.f : st[k];
  const float b = bias ? bias[c] : 0.f;
  for (int t = 0; t < n; ++t) {
    win[TAPS - 1] = __bfloat162float(x[(size_t)(q0 + t) * x_ld + c]);
    float y = b;
#pragma unroll
    for (int k = 0; k < TAPS; ++k) y += win[k] * wk[k];
    if (activation) y = mb::silu(y);
    if (write_out) out[(size_t)(q0 + t) * C + c] = y;
#pragma unroll
    for (int k = 0; k < TAPS - 1; ++k) win[k] = win[k + 1];
  }
  if (write_state) {
#pragma unroll
    for (int k = 0; k < TAPS - 1; ++k) st[k] = win[k];
  }
}

// Time-parallel form for prefill chunks: grid (channel blocks, time blocks of kConvTb tokens, sequences).
// A thread owns one channel of one time block: it primes its window from the three inputs in front
// of the block (the stored state for the first block of a continued sequence, zeros for a fresh one)
// and slides over its tokens, so every input is read once (plus the halo). The state is advanced by
// conv1d_state_kernel afterwards (stream order keeps it from racing with the first block's reads).
constexpr int kConvTb = 64;
template <int TAPS>
__global__ void __launch_bounds__(128)
conv1d_par_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, int C, const float* __restrict__ w,
                  const float* __restrict__ bias, const float* __restrict__ state, float* __restrict__ out,
                  SeqMeta sm, int activation, uint32_t* status) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int seq = blockIdx.z;
  if (c >= C) return;
  const int n = sm.q_len[seq];
  const int t0 = blockIdx.y * kConvTb;
  if (t0 >= n) return;
  const int q0 = sm.q_start[seq];
  const int slot = sm.state_slots[seq];
  if (slot < 0 || slot >= sm.num_slots) {
    if (status) atomicCAS(status, 0u, MB_ST_BOUNDS);
    return;
  }
  float win[TAPS], wk[TAPS];
#pragma unroll
  for (int k = 0; k < TAPS; ++k) wk[k] = w[(size_t)c * TAPS + k];
  const float* st = state + ((size_t)slot * C + c) * (TAPS - 1);
  const bool fresh = sm.positions[q0] == 0;
#pragma unroll
  for (int k = 0; k < TAPS - 1; ++k) {
    const int t = t0 - (TAPS - 1) + k;                   // input index of window slot k
    if (t >= 0) win[k] = __bfloat162float(x[(size_t)(q0 + t) * x_ld + c]);
    else win[k] = fresh ? 0.f : st[(TAPS - 1) + t];       // t in [-(TAPS-1), -1] -> stored input TAPS-1+t
  }
  const float b = bias ? bias[c] : 0.f;
  const int t1 = min(n, t0 + kConvTb);
  for (int t = t0; t < t1; ++t) {
    win[TAPS - 1] = __bfloat162float(x[(size_t)(q0 + t) * x_ld + c]);
    float y = b;
#pragma unroll
    for (int k = 0; k < TAPS; ++k) y += win[k] * wk[k];
    if (activation) y = mb::silu(y);
    out[(size_t)(q0 + t) * C + c] = y;
#pragma unroll
    for (int k = 0; k < TAPS - 1; ++k) win[k] = win[k + 1];
  }
}

// new state = the last TAPS - 1 inputs of (old state | this step's inputs); one thread per channel
template <int TAPS>
__global__ void __launch_bounds__(128)
conv1d_state_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, int C, float* __restrict__ state, SeqMeta sm) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int seq = blockIdx.y;
  if (c >= C) return;
  const int n = sm.q_len[seq];
  if (n <= 0) return;
  const int q0 = sm.q_start[seq];
  const int slot = sm.state_slots[seq];
  if (slot < 0 || slot >= sm.num_slots) return;
  float* st = state + ((size_t)slot * C + c) * (TAPS - 1);
  const bool fresh = sm.positions[q0] == 0;
  float nw[TAPS - 1];
#pragma unroll
  for (int k = 0; k < TAPS - 1; ++k) {
    const int t = n - (TAPS - 1) + k;                    // input index of new state slot k
    if (t >= 0) nw[k] = __bfloat162float(x[(size_t)(q0 + t) * x_ld + c]);
    else nw[k] = fresh ? 0.f : st[(TAPS - 1) + t];
  }
#pragma unroll
  for (int k = 0; k < TAPS - 1; ++k) st[k] = nw[k];
}

// ------------------------------------------------------------------ gated delta net
// grid (v_heads, num_seqs), block = DV threads. conv [T, 2 QK + V] fp32 (q | k | v),
// ba [T, 2 v_heads] fp32 (b | a), state [slots, v_heads, DK, DV] fp32, out [T, v_heads * DV].
template <int DK, int DV>
__global__ void __launch_bounds__(DV)
gdn_kernel(const float* __restrict__ conv, const float* __restrict__ ba, const float* __restrict__ A_log,
           const float* __restrict__ dt_bias, float* __restrict__ state, float* __restrict__ out,
           int k_heads, int v_heads, SeqMeta sm, int write_state, int write_out, uint32_t* status) {
  __shared__ float s_q[DK], s_k[DK];
  __shared__ float s_red[8];
  const int vh = blockIdx.x, seq = blockIdx.y, v = threadIdx.x;
  const int n = sm.q_len[seq];
  if (n <= 0) return;
  const int q0 = sm.q_start[seq];
  const int slot = sm.state_slots[seq];
  if (slot < 0 || slot >= sm.num_slots) {
    if (status && v == 0) atomicCAS(status, 0u, MB_ST_BOUNDS);
    return;
  }
  const int kh = vh / (v_heads / k_heads);
  const int QK = k_heads * DK, V = v_heads * DV;
  const int row_ld = 2 * QK + V;
  float h[DK];
  float* hs = state + (((size_t)slot * v_heads + vh) * DK) * DV + v;
  const bool fresh = sm.positions[q0] == 0;
#pragma unroll
  for (int k = 0; k < DK; ++k) h[k] = fresh ? 0.f : hs[(size_t)k * DV];
  const float a_exp = __expf(fminf(A_log[vh], 20.f));
  const float dtb = dt_bias[vh];
  const float inv_sqrt_dk = rsqrtf((float)DK);
  constexpr int NW = DV / 32;
  for (int t = 0; t < n; ++t) {
    const float* row = conv + (size_t)(q0 + t) * row_ld;
    // stage q, k of this key head and their squared norms
    __syncthreads();                                   // everyone is done with last token's s_q / s_k
    float sq = 0.f, sk = 0.f;
    for (int k = v; k < DK; k += DV) {
      const float qv = row[kh * DK + k], kv = row[QK + kh * DK + k];
      s_q[k] = qv;
      s_k[k] = kv;
      sq += qv * qv;
      sk += kv * kv;
    }
    sq = mb::warp_sum(sq);
    sk = mb::warp_sum(sk);
    if ((v & 31) == 0) { s_red[v >> 5] = sq; s_red[4 + (v >> 5)] = sk; }
    __syncthreads();
    float tq = 0.f, tk = 0.f;
#pragma unroll
    for (int wdx = 0; wdx < NW; ++wdx) { tq += s_red[wdx]; tk += s_red[4 + wdx]; }
    const float nq = rsqrtf(tq + 1e-6f) * inv_sqrt_dk, nk = rsqrtf(tk + 1e-6f);
    const float bb = ba[(size_t)(q0 + t) * 2 * v_heads + vh];
    const float aa = ba[(size_t)(q0 + t) * 2 * v_heads + v_heads + vh];
    const float sp = log1pf(__expf(fminf(aa + dtb, 20.f)));
    const float gdec = __expf(-a_exp * sp);
    const float beta = 1.f / (1.f + __expf(-bb));
    const float vv = row[2 * QK + vh * DV + v];
    float hk = 0.f;
#pragma unroll
    for (int k = 0; k < DK; ++k) hk += h[k] * s_k[k];
    hk *= nk;
    const float vp = (vv - gdec * hk) * beta;
    float o = 0.f;
#pragma unroll
    for (int k = 0; k < DK; ++k) {
      h[k] = gdec * h[k] + (s_k[k] * nk) * vp;
      o += h[k] * s_q[k];
    }
    if (write_out) out[(size_t)(q0 + t) * V + vh * DV + v] = o * nq;
  }
  if (write_state) {
#pragma unroll
    for (int k = 0; k < DK; ++k) hs[(size_t)k * DV] = h[k];
  }
}

// ------------------------------------------------------------------ mamba2
// grid (heads, num_seqs), block = 2 * P threads: thread (p, half) owns h[p, half*NH .. +NH).
// xbc [T, inner + 2 G N] fp32 (x | B | C), dt [T, dt_ld] bf16 raw, state [slots, H, P, N] fp32.
template <int NH>
__global__ void __launch_bounds__(256)
mamba2_kernel(const float* __restrict__ xbc, const __nv_bfloat16* __restrict__ dt, long long dt_ld,
              const float* __restrict__ A_log, const float* __restrict__ Dp, const float* __restrict__ dt_bias,
              float* __restrict__ state, float* __restrict__ out, int H, int G, int P, SeqMeta sm,
              int write_state, int write_out, uint32_t* status) {
  constexpr int N = 2 * NH;
  __shared__ float s_B[N], s_C[N];
  const int hd = blockIdx.x, seq = blockIdx.y;
  const int p = threadIdx.x >> 1, half = threadIdx.x & 1;
  const int n = sm.q_len[seq];
  if (n <= 0) return;
  const int q0 = sm.q_start[seq];
  const int slot = sm.state_slots[seq];
  if (slot < 0 || slot >= sm.num_slots) {
    if (status && threadIdx.x == 0) atomicCAS(status, 0u, MB_ST_BOUNDS);
    return;
  }
  const int inner = H * P, GN = G * N;
  const int grp = hd / (H / G);
  const int ld = inner + 2 * GN;
  float h[NH];
  float* hs = state + ((((size_t)slot * H + hd) * P + p) * N) + half * NH;
  const bool fresh = sm.positions[q0] == 0;
#pragma unroll
  for (int j = 0; j < NH; ++j) h[j] = fresh ? 0.f : hs[j];
  const float a_exp = __expf(A_log[hd]);
  const float dcoef = Dp[hd], dtb = dt_bias[hd];
  for (int t = 0; t < n; ++t) {
    const float* row = xbc + (size_t)(q0 + t) * ld;
    __syncthreads();
    for (int j = threadIdx.x; j < N; j += blockDim.x) {
      s_B[j] = row[inner + grp * N + j];
      s_C[j] = row[inner + GN + grp * N + j];
    }
    __syncthreads();
    const float raw = __bfloat162float(dt[(size_t)(q0 + t) * dt_ld + hd]) + dtb;
    const float dtv = raw > 20.f ? raw : log1pf(__expf(raw));
    const float dA = __expf(-a_exp * dtv);
    const float xv = row[hd * P + p];
    const float dx = dtv * xv;
    float y = 0.f;
#pragma unroll
    for (int j = 0; j < NH; ++j) {
      h[j] = dA * h[j] + dx * s_B[half * NH + j];
      y += h[j] * s_C[half * NH + j];
    }
    y += __shfl_xor_sync(0xffffffffu, y, 1);
    if (half == 0 && write_out) out[(size_t)(q0 + t) * inner + hd * P + p] = y + dcoef * xv;
  }
  if (write_state) {
#pragma unroll
    for (int j = 0; j < NH; ++j) hs[j] = h[j];
  }
}

}  // namespace

extern "C" {

int mb_causal_conv1d(const void* x, long long x_ld, int C, int taps, const float* w, const float* bias,
                     float* state, float* out, const int* q_start, const int* q_len, const int* positions,
                     const int* state_slots, int num_seqs, int num_slots, int activation, int write_state,
                     int write_out, uint32_t* status, cudaStream_t stream) {
  if (!x || !w || !state || !out || C <= 0 || num_seqs <= 0) return MB_ERR_BAD_ARG;
  SeqMeta sm{q_start, q_len, positions, state_slots, num_slots};
  dim3 grid((C + 127) / 128, num_seqs);
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  switch (taps) {
    case 2: conv1d_kernel<2><<<grid, 128, 0, stream>>>(xb, x_ld, C, w, bias, state, out, sm, activation, write_state, write_out, status); break;
    case 3: conv1d_kernel<3><<<grid, 128, 0, stream>>>(xb, x_ld, C, w, bias, state, out, sm, activation, write_state, write_out, status); break;
    case 4: conv1d_kernel<4><<<grid, 128, 0, stream>>>(xb, x_ld, C, w, bias, state, out, sm, activation, write_state, write_out, status); break;
    default: return MB_ERR_UNSUPPORTED;
  }
  return (int)cudaGetLastError();
}

// Prefill form of mb_causal_conv1d: time-parallel output, then the state update (two launches).
int mb_causal_conv1d_par(const void* x, long long x_ld, int C, int taps, const float* w, const float* bias,
                         float* state, float* out, const int* q_start, const int* q_len, const int* positions,
                         const int* state_slots, int num_seqs, int num_slots, int max_q_len, int activation,
                         int write_state, uint32_t* status, cudaStream_t stream) {
  if (!x || !w || !state || !out || C <= 0 || num_seqs <= 0 || max_q_len <= 0) return MB_ERR_BAD_ARG;
  SeqMeta sm{q_start, q_len, positions, state_slots, num_slots};
  const dim3 grid((C + 127) / 128, (max_q_len + kConvTb - 1) / kConvTb, num_seqs), sgrid((C + 127) / 128, num_seqs);
  if (grid.y > 65535 || num_seqs > 65535) return MB_ERR_TOO_LARGE;
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  switch (taps) {
    case 2:
      conv1d_par_kernel<2><<<grid, 128, 0, stream>>>(xb, x_ld, C, w, bias, state, out, sm, activation, status);
      if (write_state) conv1d_state_kernel<2><<<sgrid, 128, 0, stream>>>(xb, x_ld, C, state, sm);
      break;
    case 3:
      conv1d_par_kernel<3><<<grid, 128, 0, stream>>>(xb, x_ld, C, w, bias, state, out, sm, activation, status);
      if (write_state) conv1d_state_kernel<3><<<sgrid, 128, 0, stream>>>(xb, x_ld, C, state, sm);
      break;
    case 4:
      conv1d_par_kernel<4><<<grid, 128, 0, stream>>>(xb, x_ld, C, w, bias, state, out, sm, activation, status);
      if (write_state) conv1d_state_kernel<4><<<sgrid, 128, 0, stream>>>(xb, x_ld, C, state, sm);
      break;
    default: return MB_ERR_UNSUPPORTED;
  }
  return (int)cudaGetLastError();
}

int mb_gdn_recurrence(const float* conv, const float* ba, const float* A_log, const float* dt_bias,
                      float* state, float* out, int k_heads, int v_heads, int k_dim, int v_dim,
                      const int* q_start, const int* q_len, const int* positions, const int* state_slots,
                      int num_seqs, int num_slots, int write_state, int write_out, uint32_t* status,
                      cudaStream_t stream) {
  if (!conv || !ba || !state || !out || num_seqs <= 0 || v_heads % k_heads) return MB_ERR_BAD_ARG;
  SeqMeta sm{q_start, q_len, positions, state_slots, num_slots};
  dim3 grid(v_heads, num_seqs);
  if (k_dim == 128 && v_dim == 128)
    gdn_kernel<128, 128><<<grid, 128, 0, stream>>>(conv, ba, A_log, dt_bias, state, out, k_heads, v_heads, sm, write_state, write_out, status);
  else if (k_dim == 64 && v_dim == 64)
    gdn_kernel<64, 64><<<grid, 64, 0, stream>>>(conv, ba, A_log, dt_bias, state, out, k_heads, v_heads, sm, write_state, write_out, status);
  else if (k_dim == 32 && v_dim == 32)
    gdn_kernel<32, 32><<<grid, 32, 0, stream>>>(conv, ba, A_log, dt_bias, state, out, k_heads, v_heads, sm, write_state, write_out, status);
  else
    return MB_ERR_UNSUPPORTED;
  return (int)cudaGetLastError();
}

int mb_mamba2_scan(const float* xbc, const void* dt, long long dt_ld, const float* A_log, const float* D,
                   const float* dt_bias, float* state, float* out, int H, int G, int P, int N,
                   const int* q_start, const int* q_len, const int* positions, const int* state_slots,
                   int num_seqs, int num_slots, int write_state, int write_out, uint32_t* status,
                   cudaStream_t stream) {
  if (!xbc || !dt || !state || !out || num_seqs <= 0 || H % G || P > 128 || P <= 0) return MB_ERR_BAD_ARG;
  SeqMeta sm{q_start, q_len, positions, state_slots, num_slots};
  dim3 grid(H, num_seqs);
  const __nv_bfloat16* dtb = reinterpret_cast<const __nv_bfloat16*>(dt);
  const int threads = 2 * P;
  if (N == 128)
    mamba2_kernel<64><<<grid, threads, 0, stream>>>(xbc, dtb, dt_ld, A_log, D, dt_bias, state, out, H, G, P, sm, write_state, write_out, status);
  else if (N == 64)
    mamba2_kernel<32><<<grid, threads, 0, stream>>>(xbc, dtb, dt_ld, A_log, D, dt_bias, state, out, H, G, P, sm, write_state, write_out, status);
  else if (N == 16)
    mamba2_kernel<8><<<grid, threads, 0, stream>>>(xbc, dtb, dt_ld, A_log, D, dt_bias, state, out, H, G, P, sm, write_state, write_out, status);
  else
    return MB_ERR_UNSUPPORTED;
  return (int)cudaGetLastError();
}

}  // extern "C"
