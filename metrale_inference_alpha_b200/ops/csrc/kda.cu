// Kimi delta attention (KDA): the gated delta rule with one decay per key channel.
//
// Per head, per token, on the fp32 state S[k][v] (k the key channel, v the value channel):
//   gate[k]  = lower_bound * sigmoid(exp(A_log[h]) * (g_raw[k] + dt_bias[h, k]))      (a log-decay, <= 0)
//   S[k][v] *= exp(gate[k])
//   delta[v] = (v[v] - sum_k S[k][v] k^[k]) * sigmoid(b_raw)
//   S[k][v] += k^[k] * delta[v]
//   o[v]     = sum_k S[k][v] q^[k] / sqrt(D)              with q^, k^ the l2-normalised q, k
// and, fused behind it when the caller passes the output norm, the sigmoid-gated RMSNorm of the
// layer: y[v] = o[v] * rsqrt(mean_v(o^2) + eps) * w[v] * sigmoid(out_gate[v]), written as bf16.
//
// One launch serves every sequence of a ragged batch (decode rows, verify rows, prefill chunks):
// grid (heads, sequences), D threads; thread v keeps column S[:, v] in registers, the token's q^, k^
// and exp(gate) are staged in shared memory once per token, the l2 norms, the gate law, the beta
// sigmoid and the output norm all live in this kernel (the reference runs them as separate launches:
// kernels/gb10/common/kda_gate.cu, kda_recurrent.cu, kda_layer_ops.cu::kda_o_norm_gated_bf16, with
// l2_norm fused into its decode conv).
#include "common.cuh"

namespace {

struct KdaSeqs {
  const int* q_start;
  const int* q_len;
  const int* positions;
  const int* state_slots;
  int num_slots;
};

struct KdaArgs {
  const float* conv;        // [T, 3 H D]  q | k | v after conv + SiLU
  const float* g_raw;       // [T, H D]
  const float* b_raw;       // [T, b_ld], head h at column h
  int b_ld;
  const float* A_log;       // [H]
  const float* dt_bias;     // [H D]
  float lower_bound;
  float* state;             // [slots, H, D, D]
  float* out;               // [T, H D] fp32 or null
  __nv_bfloat16* out_norm;  // [T, H D] bf16 or null (needs norm_w and out_gate)
  const __nv_bfloat16* out_gate;   // [T, gate_ld]
  long long gate_ld;
  const float* norm_w;      // [D]
  float eps;
  int H;
  KdaSeqs sm;
  int write_state, write_out;
  uint32_t* status;
};

template <int D>
__global__ void __launch_bounds__(D) kda_kernel(const KdaArgs a) {
  __shared__ __align__(16) float s_q[D], s_k[D], s_g[D];
  __shared__ float s_red[3][4];
  const int hd = blockIdx.x, seq = blockIdx.y, v = threadIdx.x;
  const int n = a.sm.q_len[seq];
  if (n <= 0) return;
  const int q0 = a.sm.q_start[seq];
  const int slot = a.sm.state_slots[seq];
  if (slot < 0 || slot >= a.sm.num_slots) {
    if (a.status && v == 0) atomicCAS(a.status, 0u, MB_ST_BOUNDS);
    return;
  }
  constexpr int NW = D / 32;
  const int HD = a.H * D;
  float h[D];
  float* hs = a.state + (((size_t)slot * a.H + hd) * D) * D + v;
  const bool fresh = a.sm.positions[q0] == 0;
#pragma unroll
  for (int k = 0; k < D; ++k) h[k] = fresh ? 0.f : hs[(size_t)k * D];
  const float a_exp = __expf(fminf(a.A_log[hd], 20.f));
  const float dtb = a.dt_bias[hd * D + v];
  const float scale = rsqrtf((float)D);
  const float nw = a.norm_w ? a.norm_w[v] : 1.f;
  // the next token's inputs are fetched while the current token is computed (a prefill walks thousands of
  // tokens with one warp per scheduler: a global load in the dependent chain of every token would set the pace)
  float n_q, n_k, n_v, n_g, n_b, n_og = 0.f;
  auto fetch = [&](int t) {
    const size_t row = (size_t)(q0 + t);
    const float* cr = a.conv + row * 3 * HD;
    n_q = cr[hd * D + v];
    n_k = cr[HD + hd * D + v];
    n_v = cr[2 * HD + hd * D + v];
    n_g = a.g_raw[row * HD + hd * D + v];
    n_b = a.b_raw[row * a.b_ld + hd];
    if (a.out_norm && a.write_out) n_og = __bfloat162float(a.out_gate[row * a.gate_ld + hd * D + v]);
  };
  fetch(0);
  for (int t = 0; t < n; ++t) {
    const size_t row = (size_t)(q0 + t);
    __syncthreads();                                    // the last token's shared values are consumed
    const float qv = n_q, kv = n_k, vv = n_v, braw = n_b, og = n_og;
    const float gate = a.lower_bound / (1.f + __expf(-a_exp * (n_g + dtb)));
    if (t + 1 < n) fetch(t + 1);
    s_q[v] = qv;
    s_k[v] = kv;
    s_g[v] = __expf(gate);
    const float sq = mb::warp_sum(qv * qv), sk = mb::warp_sum(kv * kv);
    if ((v & 31) == 0) {
      s_red[0][v >> 5] = sq;
      s_red[1][v >> 5] = sk;
    }
    __syncthreads();
    float tq = 0.f, tk = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      tq += s_red[0][w];
      tk += s_red[1][w];
    }
    const float nq = rsqrtf(tq + 1e-6f) * scale, nk = rsqrtf(tk + 1e-6f);
    const float beta = 1.f / (1.f + __expf(-braw));
    // four partial sums per reduction: with one warp per scheduler the dependent fma chain is the limit
    float hk4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < D; k += 4) {
      const float4 g4 = *reinterpret_cast<const float4*>(&s_g[k]);
      const float4 k4 = *reinterpret_cast<const float4*>(&s_k[k]);
      h[k] *= g4.x;
      h[k + 1] *= g4.y;
      h[k + 2] *= g4.z;
      h[k + 3] *= g4.w;
      hk4[0] = fmaf(h[k], k4.x, hk4[0]);
      hk4[1] = fmaf(h[k + 1], k4.y, hk4[1]);
      hk4[2] = fmaf(h[k + 2], k4.z, hk4[2]);
      hk4[3] = fmaf(h[k + 3], k4.w, hk4[3]);
    }
    const float hk = (hk4[0] + hk4[1]) + (hk4[2] + hk4[3]);
    const float delta = (vv - hk * nk) * beta * nk;      // the second nk belongs to k^ in the update
    float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < D; k += 4) {
      const float4 k4 = *reinterpret_cast<const float4*>(&s_k[k]);
      const float4 q4 = *reinterpret_cast<const float4*>(&s_q[k]);
      h[k] = fmaf(k4.x, delta, h[k]);
      h[k + 1] = fmaf(k4.y, delta, h[k + 1]);
      h[k + 2] = fmaf(k4.z, delta, h[k + 2]);
      h[k + 3] = fmaf(k4.w, delta, h[k + 3]);
      o4[0] = fmaf(h[k], q4.x, o4[0]);
      o4[1] = fmaf(h[k + 1], q4.y, o4[1]);
      o4[2] = fmaf(h[k + 2], q4.z, o4[2]);
      o4[3] = fmaf(h[k + 3], q4.w, o4[3]);
    }
    float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
    o *= nq;
    if (a.write_out) {
      if (a.out) a.out[row * HD + hd * D + v] = o;
      if (a.out_norm) {
        const float so = mb::warp_sum(o * o);
        if ((v & 31) == 0) s_red[2][v >> 5] = so;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) tot += s_red[2][w];
        a.out_norm[row * HD + hd * D + v] =
            __float2bfloat16(o * rsqrtf(tot / D + a.eps) * nw / (1.f + __expf(-og)));
      }
    }
  }
  if (a.write_state) {
#pragma unroll
    for (int k = 0; k < D; ++k) hs[(size_t)k * D] = h[k];
  }
}

}  // namespace

struct MbKdaArgs {
  const void* conv;
  const void* g_raw;
  const void* b_raw;
  int b_ld;
  const void* A_log;
  const void* dt_bias;
  float lower_bound;
  void* state;
  void* out;
  void* out_norm;
  const void* out_gate;
  long long gate_ld;
  const void* norm_w;
  float eps;
  int H, D;
  const void* q_start;
  const void* q_len;
  const void* positions;
  const void* state_slots;
  int num_seqs, num_slots, write_state, write_out;
  void* status;
};

extern "C" int mb_kda_recurrence(const MbKdaArgs* p, cudaStream_t stream) {
  if (!p || !p->conv || !p->g_raw || !p->b_raw || !p->state || p->num_seqs <= 0 || p->H <= 0) return MB_ERR_BAD_ARG;
  if (p->out_norm && (!p->norm_w || !p->out_gate)) return MB_ERR_BAD_ARG;
  KdaArgs a{static_cast<const float*>(p->conv), static_cast<const float*>(p->g_raw),
            static_cast<const float*>(p->b_raw), p->b_ld, static_cast<const float*>(p->A_log),
            static_cast<const float*>(p->dt_bias), p->lower_bound, static_cast<float*>(p->state),
            static_cast<float*>(p->out), static_cast<__nv_bfloat16*>(p->out_norm),
            static_cast<const __nv_bfloat16*>(p->out_gate), p->gate_ld, static_cast<const float*>(p->norm_w),
            p->eps, p->H,
            KdaSeqs{static_cast<const int*>(p->q_start), static_cast<const int*>(p->q_len),
                    static_cast<const int*>(p->positions), static_cast<const int*>(p->state_slots), p->num_slots},
            p->write_state, p->write_out, static_cast<uint32_t*>(p->status)};
  const dim3 grid(p->H, p->num_seqs);
  if (p->D == 128) kda_kernel<128><<<grid, 128, 0, stream>>>(a);
  else if (p->D == 64) kda_kernel<64><<<grid, 64, 0, stream>>>(a);
  else if (p->D == 32) kda_kernel<32><<<grid, 32, 0, stream>>>(a);
  else return MB_ERR_UNSUPPORTED;
  return (int)cudaGetLastError();
}
