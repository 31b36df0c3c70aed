// Weight-stationary ("swap-AB") linear layer for sm_100a:
//     out[m, n] = epilogue( sum_k X[m, k] * W[n, k] )
// The weight tile is the UMMA "A" operand (M = 128 output features per CTA) and
// the activation tile is the "B" operand (UMMA N = TN tokens, 16..256), so decode
// batches of 1..128 tokens waste no tensor work and each CTA streams a
// [128 x K] slab of weights exactly once through a TMA -> shared -> tcgen05.mma
// pipeline with the fp32 accumulator in TMEM.
//
// Operand kinds
//   KIND_BF16   W, X bf16                    tcgen05.mma kind::f16
//   KIND_FP8    W, X e4m3; per-row weight scale and per-token activation scale
//               applied in the epilogue      tcgen05.mma kind::f8f6f4
//   KIND_NVFP4  W, X packed e2m1 (two per byte, even k in the low nibble) with
//               per-16 ue4m3 scale factors staged smem -> TMEM by tcgen05.cp and
//               an fp32 global scale (x per-token activation scale) in the
//               epilogue                     kind::mxf4nvf4.block_scale.scale_vec::4X
//   KIND_FP8_BLOCK  W e4m3 with one fp32 scale per 128x128 block, X e4m3 with one
//               scale per token per 128-wide k group: each 128-deep k block is
//               accumulated into one of two TMEM buffers and promoted into fp32
//               registers by the epilogue warps with both scales applied.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (one TMEM lane quadrant each).
//
// Small-N layers (o_proj, down_proj) use split-K over blockIdx.z: every split
// writes an fp32 partial tile to a caller-provided workspace, bumps a per-tile
// counter, and the last arriver sums the partials in split order (deterministic)
// and runs the epilogue; it also re-zeroes the counter so no memset is needed
// between launches.
//
// Reference behaviour covered: the projection GEMM/GEMV tiers of
// kernels/gb10/common/{dense_gemm_bf16,dense_gemv_bf16*,w4a16_gemm,w4a16_gemv,
// w8a16_gemm*,w8a8_gemv,fp8_gemm_t_blockscaled}.cu and the W4A4 path of
// kernels/gb10/qwen3.6-27b/nvfp4/nvfp4_mmq.cu (compiled out for sm_100a there).
#include "common.cuh"
#include "gemm_args.h"
#include <mutex>
#include "tensormap.h"
#include "noalloc.h"

namespace {

enum { KIND_BF16 = 0, KIND_FP8 = 1, KIND_NVFP4 = 2, KIND_FP8_BLOCK = 3 };
enum { EPI_PLAIN = 0, EPI_SWIGLU = 1 };

struct GemmParams {
  int M, N, K, ldo;
  void* out;
  const __nv_bfloat16* residual;
  const float* w_scale;   // KIND_FP8: [N]; KIND_NVFP4: optional per-row global scale [N]; KIND_FP8_BLOCK: [ceil(N/128), ceil(K/128)]
  const float* a_scale;   // KIND_FP8 / NVFP4: [M] or null; KIND_FP8_BLOCK: [ceil(K/128), a_ld]
  int a_ld;
  float alpha;
  const uint8_t* sfa;     // NVFP4 tiled scale factors of W: [ceil(N/128)][k64 groups][512]
  const uint8_t* sfb;     // NVFP4 tiled scale factors of X: [ceil(M/128)][k64 groups][512]
  int sf_k64;             // number of 64-element k groups allocated per 128-row block
  float* ws;
  uint32_t* cnt;
  int splits, kb_per_split, num_kb;
  int epilogue, out_f32;
  uint32_t* status;
  // grouped (MoE) mode: blockIdx.y indexes a tile work-list; W is [experts * n_per_expert, K]
  const int* tile_expert;
  const int* tile_row0;
  const int* tile_nrows;
  int n_per_expert;
  // quantised output of the SwiGLU epilogue (persistent kernel): packed e2m1 + tiled ue4m3 scale
  // factors for the consuming W4A4 GEMM, with a calibrated (static) global scale
  uint8_t* outq;      // [M, ldq] bytes, two values per byte; null = bf16 / fp32 output
  int ldq;
  uint8_t* outq_sf;   // [ceil(M / 128)][outq_sf_k64][512]
  int outq_sf_k64;
  float outq_gs;
  int m_fastest;      // token tiles in blockIdx.x (prefill): see the kernel's launch-order note
  int cluster;        // splits form a thread-block cluster (co-resident, one cluster barrier instead of counters)
  int cluster_ws;     // with `cluster`: partial tiles are exchanged through the global workspace (L2), which
                      // measures ~4x faster than distributed shared memory for 64 KB tiles; 0 = over DSMEM
#ifdef MB_GEMM_TIMING_EXPERIMENTS
  // kernel-development builds only (never the shipped library): per-phase cycle stamps of CTA
  // (0,0,0) and the last CTA in x, and switches that skip parts of the work to time the rest
  long long* trace;
  int dbg;   // 1 skip SF copies, 2 skip epilogue stores, 4 skip MMAs, 8 skip SF loads, 32 stale activation tiles
#endif
};

constexpr int kTileN = 128;  // output features per CTA (UMMA M)

template <int KIND, int TN, int CTAS = 1>
struct Cfg {
  static constexpr int kABytes = kTileN * 128;
  static constexpr int kBBytes = TN * 128;
  static constexpr int kSfBytes = (KIND == KIND_NVFP4) ? 2048 : 0;
  static constexpr int kStageBytes = kABytes + kBBytes + 2 * kSfBytes;
  // one CTA per SM with a deep pipeline: two co-resident CTAs with half the stages measured
  // slower on the decode shapes (fewer bytes in flight per CTA on the split-K GEMMs). CTAS = 2 is
  // for the grouped (MoE) work lists of small token tiles: thousands of CTAs of 3 - 8 k blocks each,
  // where a second resident CTA runs its main loop under the first one's prologue and epilogue.
  static constexpr int kCtasPerSm = CTAS;
  static constexpr int kBudget = (CTAS == 2 ? 100 : 200) * 1024;
  static constexpr int kStagesRaw = kBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kAccCols = (KIND == KIND_FP8_BLOCK) ? 2 * TN : TN;
  static constexpr int kNeedCols = kAccCols + (KIND == KIND_NVFP4 ? 64 : 0);   // 2 x (SFA 16 + SFB 16)
  static constexpr int kTmemCols =
      kNeedCols <= 32 ? 32 : kNeedCols <= 64 ? 64 : kNeedCols <= 128 ? 128 : kNeedCols <= 256 ? 256 : 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
};

#ifdef MB_GEMM_TIMING_EXPERIMENTS
#define MB_STAMP(i)                                                                              \
  do {                                                                                           \
    if (p.trace && blockIdx.y == 0 && blockIdx.x == 0 && (blockIdx.z == 0 || blockIdx.z == gridDim.z - 1)) \
      p.trace[(blockIdx.z == 0 ? 0 : 12) + (i)] = clock64();                                     \
  } while (0)
#define MB_DBG(bit) (p.dbg & (bit))
#else
#define MB_STAMP(i) do { } while (0)
#define MB_DBG(bit) 0
#endif

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int KIND, int TN, int CTAS = 1>
__global__ void __launch_bounds__(192, CTAS)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const GemmParams p) {
  using C = Cfg<KIND, TN, CTAS>;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int is_last_s;
  __shared__ float s_ascale[TN];

  const int warp = threadIdx.x >> 5;
  // Launch order: blockIdx.x runs fastest. Decode (one token tile) walks the weight tiles in x. With
  // many token tiles (prefill) the token tiles go in x instead, so the CTAs that are resident together
  // share a few weight tiles (each read from DRAM once and re-served from L2) rather than streaming
  // the whole weight matrix once per token tile.
  const int tile_n = p.m_fastest ? blockIdx.y : blockIdx.x;
  const int tile_m = p.m_fastest ? blockIdx.x : blockIdx.y;
  const int split = blockIdx.z;
  const int tiles_n_grid = p.m_fastest ? gridDim.y : gridDim.x;
  int m_row0 = tile_m * TN, m_end = p.M, expert = 0, n_limit = p.N;
  if (p.tile_expert) {
    mb::pdl_wait();                               // the work list is written by the preceding sort kernel
    expert = p.tile_expert[tile_m];
    if (expert < 0) return;                       // unused work-list entry (uniform for the CTA)
    m_row0 = p.tile_row0[tile_m];
    m_end = m_row0 + p.tile_nrows[tile_m];
    n_limit = p.n_per_expert;
  }
  const int w_row0 = expert * p.n_per_expert + tile_n * kTileN;   // n_per_expert = 0 when not grouped
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
  const int nkb = kb1 - kb0;

  if (threadIdx.x == 0) MB_STAMP(0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mb::mbar_init(&full_bar[s], 1);
      mb::mbar_init(&empty_bar[s], 1);
    }
    mb::mbar_init(&acc_full[0], 1);
    mb::mbar_init(&acc_full[1], 1);
    mb::mbar_init(&acc_empty[0], 128);
    mb::mbar_init(&acc_empty[1], 128);
    mb::mbar_fence_init();
    mb::tma_prefetch_desc(&tmA);
    mb::tma_prefetch_desc(&tmB);
  }
  if (warp == 1) mb::tmem_alloc(&tmem_base_s, C::kTmemCols);
  mb::tc_fence_before();
  __syncthreads();
  mb::tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  // Programmatic dependent launch: everything above touched no global memory. The weights are
  // never written by a kernel of the same stream, so the producer starts streaming them before
  // the wait; only the activation operand, its scale factors and the epilogue's reads and
  // writes wait for the preceding kernel.
  mb::pdl_launch_dependents();
  if (threadIdx.x == 0) MB_STAMP(1);

  auto sA = [&](int s) { return smem + s * C::kStageBytes; };
  auto sB = [&](int s) { return smem + s * C::kStageBytes + C::kABytes; };
  auto sSFA = [&](int s) { return smem + s * C::kStageBytes + C::kABytes + C::kBBytes; };
  auto sSFB = [&](int s) {
    return smem + s * C::kStageBytes + C::kABytes + C::kBBytes + C::kSfBytes;
  };
  // inner TMA coordinate advance per k block, in tensor-map elements
  constexpr int kCoordStep = (KIND == KIND_BF16) ? 64 : 128;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (mb::elect_one()) {
      const bool sf_load = (KIND == KIND_NVFP4) && !MB_DBG(8);
      const uint32_t stage_tx = C::kStageBytes - (KIND == KIND_NVFP4 && !sf_load ? 4096 : 0);
      auto load_w = [&](int i) {                   // weight tile + its scale factors
        const int s = i % kStages, kb = kb0 + i;
        mb::tma_load_2d(sA(s), &tmA, &full_bar[s], kb * kCoordStep, w_row0);
        if (sf_load)
          mb::bulk_load(sSFA(s), p.sfa + ((size_t)(w_row0 / kTileN) * p.sf_k64 + (size_t)kb * 4) * 512, 2048, &full_bar[s]);
      };
      auto load_x = [&](int i) {                   // activation tile + its scale factors
        const int s = i % kStages, kb = kb0 + i;
        mb::tma_load_2d(sB(s), &tmB, &full_bar[s], kb * kCoordStep, m_row0);
        if (sf_load)
          mb::bulk_load(sSFB(s), p.sfb + ((size_t)(m_row0 / 128) * p.sf_k64 + (size_t)kb * 4) * 512, 2048,
                        &full_bar[s]);
      };
      const int pre = min(nkb, kStages);           // the first round needs no empty-slot wait
      for (int i = 0; i < pre; ++i) {
        mb::mbar_expect_tx(&full_bar[i], stage_tx);
        load_w(i);
      }
      mb::pdl_wait();
      for (int i = 0; i < pre; ++i) {
        load_x(i);
        if (i == 0) MB_STAMP(2);
      }
      for (int i = pre; i < nkb; ++i) {
        const int s = i % kStages;
        const uint32_t ph = (i / kStages) & 1;
        if (!mb::mbar_wait(&empty_bar[s], ph ^ 1, p.status, MB_ST_TIMEOUT_TMA)) break;
        mb::mbar_expect_tx(&full_bar[s], stage_tx);
        load_w(i);
        load_x(i);
      }
    }
    __syncwarp();
    if (p.cluster) { mb::cluster_sync_all(); if (!p.cluster_ws) mb::cluster_sync_all(); }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (mb::elect_one()) {
      uint32_t idesc;
      if constexpr (KIND == KIND_BF16) idesc = mb::umma_idesc(1, 1, kTileN, TN);
      else if constexpr (KIND == KIND_NVFP4) idesc = mb::umma_idesc_bs(1, 1, kTileN, TN, 0);
      else idesc = mb::umma_idesc(0, 0, kTileN, TN);
      // scale factors alternate between two TMEM column sets so the copies of k block i + 1
      // do not wait for the MMAs of k block i to release the columns
      constexpr uint32_t kSfBase = TN;
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % kStages;
        const uint32_t ph = (i / kStages) & 1;
        uint32_t acc = tmem;
        if constexpr (KIND == KIND_FP8_BLOCK) {
          const int buf = i & 1;
          const uint32_t aph = (i >> 1) & 1;
          ok = mb::mbar_wait(&acc_empty[buf], aph ^ 1, p.status, MB_ST_TIMEOUT_MMA);
          if (!ok) break;
          acc = tmem + buf * TN;
        }
        ok = mb::mbar_wait(&full_bar[s], ph, p.status, MB_ST_TIMEOUT_MMA);
        if (!ok) break;
        mb::tc_fence_after();
        if (i == 0) MB_STAMP(3);
        const uint32_t a_base = mb::smem_u32(sA(s)), b_base = mb::smem_u32(sB(s));
        const uint32_t kSfaCol = kSfBase + (i & 1) * 32, kSfbCol = kSfaCol + 16;
        if constexpr (KIND == KIND_NVFP4) {
          if (!MB_DBG(1)) {
            const uint32_t sfa = mb::smem_u32(sSFA(s)), sfb = mb::smem_u32(sSFB(s));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              mb::tmem_cp_sf(tmem + kSfaCol + j * 4, mb::umma_desc_sf(sfa + j * 512));
              mb::tmem_cp_sf(tmem + kSfbCol + j * 4, mb::umma_desc_sf(sfb + j * 512));
            }
          }
        }
        if (!MB_DBG(4)) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint64_t da = mb::umma_desc_sw128(a_base + j * 32);
          const uint64_t db = mb::umma_desc_sw128(b_base + j * 32);
          if constexpr (KIND == KIND_BF16) {
            mb::umma_f16(acc, da, db, idesc, (i | j) != 0);
          } else if constexpr (KIND == KIND_FP8) {
            mb::umma_f8f6f4(acc, da, db, idesc, (i | j) != 0);
          } else if constexpr (KIND == KIND_FP8_BLOCK) {
            mb::umma_f8f6f4(acc, da, db, idesc, j != 0);
          } else {
            mb::umma_nvfp4(acc, da, db, idesc, tmem + kSfaCol + j * 4, tmem + kSfbCol + j * 4,
                           (i | j) != 0);
          }
        }
        }
        mb::tc_commit(&empty_bar[s]);
        if constexpr (KIND == KIND_FP8_BLOCK) mb::tc_commit(&acc_full[i & 1]);
      }
      if constexpr (KIND != KIND_FP8_BLOCK) mb::tc_commit(&acc_full[0]);
      MB_STAMP(4);
    }
    __syncwarp();
    if (p.cluster) { mb::cluster_sync_all(); if (!p.cluster_ws) mb::cluster_sync_all(); }
  } else {
    // ------------------------------------------------------------ epilogue
    // (a) TMEM -> registers -> fp32 staging tile [m][n] in the (by then idle) pipeline
    //     buffers, or -> the split-K workspace; (b) barrier; (c) all 128 threads walk the
    //     tile row by row with 16-byte accesses: scales, SwiGLU, residual, store.
    const int q = warp & 3;
    const int lane = threadIdx.x & 31;
    const int et = threadIdx.x - 64;                       // 0..127
    const int m0 = m_row0;
    const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
    float* s_tile = reinterpret_cast<float*>(smem);
    bool ok = true;
    const bool swiglu = p.epilogue == EPI_SWIGLU;
    mb::pdl_wait();                                        // first global access of these warps follows
    // per-token scales of this tile, staged while the main loop runs
    for (int j = et; j < TN; j += 128) {
      float sc = 1.f;
      if constexpr (KIND == KIND_FP8 || KIND == KIND_NVFP4) {
        if (p.a_scale && m0 + j < m_end) sc = __ldg(&p.a_scale[m0 + j]);
      }
      s_ascale[j] = sc;
    }
    // this thread's fixed column group in phase (c): 8 columns (16 with SwiGLU)
    const int cpt = swiglu ? 16 : 8;
    const int tpr = kTileN / cpt;                          // threads per row
    const int col0 = (et % tpr) * cpt;
    float wcol[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float wsc = p.alpha;
      if constexpr (KIND == KIND_FP8 || KIND == KIND_NVFP4) {
        const int n = tile_n * kTileN + col0 + i;
        if (i < cpt && p.w_scale && n < n_limit) wsc *= __ldg(&p.w_scale[(size_t)expert * p.n_per_expert + n]);
      }
      wcol[i] = wsc;
    }
    const size_t tile_lin = (size_t)tile_m * tiles_n_grid + tile_n;
    float* wsp = (p.splits > 1 && (!p.cluster || p.cluster_ws)) ? p.ws + (tile_lin * p.splits + split) * (size_t)(TN * kTileN) : s_tile;

    if constexpr (KIND == KIND_FP8_BLOCK) {
      float accr[TN];
#pragma unroll
      for (int j = 0; j < TN; ++j) accr[j] = 0.f;
      const int kgroups = (p.K + 127) / 128;
      for (int i = 0; i < nkb && ok; ++i) {
        const int buf = i & 1;
        const uint32_t aph = (i >> 1) & 1;
        ok = mb::mbar_wait(&acc_full[buf], aph, p.status, MB_ST_TIMEOUT_EPI);
        if (!ok) break;
        mb::tc_fence_after();
        const int kb = kb0 + i;
        const float wsc = __ldg(&p.w_scale[((size_t)expert * (p.n_per_expert / kTileN) + tile_n) * kgroups + kb]);
        const float* as = p.a_scale + (size_t)kb * p.a_ld + m0;
#pragma unroll
        for (int c = 0; c < TN / 16; ++c) {
          float v[16];
          mb::tmem_ld16(lane_addr + buf * TN + c * 16, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) accr[c * 16 + j] += v[j] * (wsc * __ldg(&as[c * 16 + j]));
        }
        mb::tc_fence_before();
        mb::mbar_arrive(&acc_empty[buf]);
      }
      if (threadIdx.x == 64) MB_STAMP(5);
      // the last k block's MMAs are complete (acc_full observed), so the stage buffers are idle
      if (ok) {
#pragma unroll
        for (int j = 0; j < TN; ++j) wsp[j * kTileN + q * 32 + lane] = accr[j];
      }
    } else {
      ok = mb::mbar_wait(&acc_full[0], 0, p.status, MB_ST_TIMEOUT_EPI);
      if (threadIdx.x == 64) MB_STAMP(5);
      if (ok) {
        mb::tc_fence_after();
#pragma unroll 2
        for (int c = 0; c < TN / 16; ++c) {
          float v[16];
          mb::tmem_ld16(lane_addr + c * 16, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) wsp[(c * 16 + j) * kTileN + q * 32 + lane] = v[j];
        }
      }
    }
    int nsrc = 1;                                          // tiles to sum in phase (c)
    const float* src = s_tile;
    bool do_store = ok;
    int row_lo = 0, row_hi = TN;                           // rows this CTA finishes
    if (p.splits > 1 && p.cluster) {
      // every CTA of the cluster holds its partial tile in shared memory at the same offset;
      // each one finishes a contiguous share of the rows, summing the peers' tiles in split
      // order through distributed shared memory
      if (threadIdx.x == 64) MB_STAMP(8);
      if (p.cluster_ws) __threadfence();                   // partial tile in global memory: visible to the cluster's other SMs
      epi_bar_sync();
      mb::cluster_sync_all();
      if (threadIdx.x == 64) MB_STAMP(9);
      nsrc = p.splits;
      if (p.cluster_ws) src = p.ws + tile_lin * p.splits * (size_t)(TN * kTileN);
      const int share = (((TN + p.splits - 1) / p.splits) + 7) & ~7;
      row_lo = split * share;
      row_hi = min(TN, row_lo + share);
    } else if (p.splits > 1) {
      // last-arriver reduction, summed in split order so the result does not depend on
      // which CTA finishes last
      if (threadIdx.x == 64) MB_STAMP(8);
      __threadfence();
      epi_bar_sync();
      if (threadIdx.x == 64) {
        const uint32_t prev = atomicAdd(&p.cnt[tile_lin], 1u);
        const int last = (prev == (uint32_t)p.splits - 1);
        if (last) p.cnt[tile_lin] = 0;
        is_last_s = last;
      }
      epi_bar_sync();
      if (threadIdx.x == 64) MB_STAMP(9);
      do_store = do_store && is_last_s;
      if (do_store) __threadfence();
      if (threadIdx.x == 64) MB_STAMP(10);
      nsrc = p.splits;
      src = p.ws + tile_lin * p.splits * (size_t)(TN * kTileN);
    } else {
      epi_bar_sync();
    }
    if (do_store && !MB_DBG(2)) {
      const int rpp = 128 / tpr;                           // rows per pass
      const int n_out0 = swiglu ? (tile_n * kTileN + col0) / 2 : tile_n * kTileN + col0;
      const int n_out_limit = swiglu ? n_limit / 2 : n_limit;
      const bool vec_ok = (p.ldo % 8 == 0) && (n_out0 + 8 <= n_out_limit) &&
                          ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.residual)) & 15) == 0;
      const int rows_valid = min(row_hi, m_end - m0);
      const int nf4 = cpt / 4;                             // float4 per row for this thread
      // scale + (SwiGLU) + residual + store of one row held in x[]
      // `rpre`: the residual vector of this row, loaded by the caller ahead of the partial tiles so
      // that its latency overlaps theirs (null: load it here)
      auto emit = [&](int mr, const float* x, const uint4* rpre = nullptr) {
        const int m = m0 + mr;
        const float as = s_ascale[mr];
        float y[8];
        if (swiglu) {
#pragma unroll
          for (int i = 0; i < 8; ++i) y[i] = mb::silu(x[2 * i] * wcol[2 * i] * as) * (x[2 * i + 1] * wcol[2 * i + 1] * as);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) y[i] = x[i] * wcol[i] * as;
        }
        const size_t o = (size_t)m * p.ldo + n_out0;
        if (vec_ok) {
          if (p.residual) {
            const uint4 r = rpre ? *rpre : __ldg(reinterpret_cast<const uint4*>(p.residual + o));
            const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = __bfloat1622float2(rb[i]);
              y[2 * i] += f.x; y[2 * i + 1] += f.y;
            }
          }
          if (p.out_f32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o);
            dst[0] = make_float4(y[0], y[1], y[2], y[3]);
            dst[1] = make_float4(y[4], y[5], y[6], y[7]);
          } else {
            uint4 pk;
            __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int i = 0; i < 4; ++i) pb[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + o) = pk;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (n_out0 + i < n_out_limit) {
              float val = y[i];
              if (p.residual) val += __bfloat162float(p.residual[o + i]);
              if (p.out_f32) reinterpret_cast<float*>(p.out)[o + i] = val;
              else reinterpret_cast<__nv_bfloat16*>(p.out)[o + i] = __float2bfloat16(val);
            }
          }
        }
      };
      if (nsrc == 1) {
        // staged tile in shared memory
        for (int mr = row_lo + et / tpr; mr < rows_valid; mr += rpp) {
          float x[16];
          uint4 rv = make_uint4(0, 0, 0, 0);
          const bool pre = vec_ok && p.residual;
          if (pre) rv = __ldg(reinterpret_cast<const uint4*>(p.residual + (size_t)(m0 + mr) * p.ldo + n_out0));
          const float4* row = reinterpret_cast<const float4*>(s_tile + mr * kTileN + col0);
#pragma unroll
          for (int i4 = 0; i4 < 4; ++i4) {
            const float4 f = i4 < nf4 ? row[i4] : make_float4(0.f, 0.f, 0.f, 0.f);
            x[i4 * 4] = f.x; x[i4 * 4 + 1] = f.y; x[i4 * 4 + 2] = f.z; x[i4 * 4 + 3] = f.w;
          }
          emit(mr, x, pre ? &rv : nullptr);
        }
      } else if (p.cluster && p.cluster_ws) {
        // split-K cluster, partial tiles in the L2-resident workspace: this CTA's row share of
        // every split's tile is brought into the (idle) stage buffers with asynchronous 16-byte
        // copies that are all in flight together, so the ~1.3 us first-touch latency of lines
        // another SM has just written is paid once, not once per batch of register loads; the
        // rows are then summed from shared memory in split order.
        const int my_rows = rows_valid - row_lo;                       // may be <= 0
        if (my_rows > 0) {
          const int chunks_per_row = kTileN / 4;                       // 16-byte chunks
          const int per_split = my_rows * chunks_per_row;
          for (int i = et; i < nsrc * per_split; i += 128) {
            const int sI = i / per_split, rem = i - sI * per_split;
            const float* g = src + (size_t)sI * (TN * kTileN) + (size_t)row_lo * kTileN + rem * 4;
            const uint32_t d = mb::smem_u32(s_tile + (size_t)sI * per_split * 4 + rem * 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(g) : "memory");
          }
        }
        // residual vectors of this thread's first two rows: independent loads, issued under the copies
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        epi_bar_sync();
        if (threadIdx.x == 64) MB_STAMP(11);
        const int per_split_f = (my_rows > 0 ? my_rows : 0) * kTileN;
        for (int mr = row_lo + et / tpr; mr < rows_valid; mr += rpp) {
          const bool pre = vec_ok && p.residual;
          uint4 rv = make_uint4(0, 0, 0, 0);
          if (pre) rv = __ldg(reinterpret_cast<const uint4*>(p.residual + (size_t)(m0 + mr) * p.ldo + n_out0));
          float x[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) x[i] = 0.f;
          for (int sI = 0; sI < nsrc; ++sI) {
            const float4* row = reinterpret_cast<const float4*>(s_tile + (size_t)sI * per_split_f + (mr - row_lo) * kTileN + col0);
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
              if (i4 < nf4) {
                const float4 f = row[i4];
                x[i4 * 4] += f.x; x[i4 * 4 + 1] += f.y; x[i4 * 4 + 2] += f.z; x[i4 * 4 + 3] += f.w;
              }
            }
          }
          emit(mr, x, pre ? &rv : nullptr);
        }
      } else {
        // split-K: partial tiles in the workspace (L2). Two rows x all splits are requested
        // before the first use so the loads overlap; summed in split order.
        constexpr int kMaxBatch = 4;                       // splits handled per load batch
        for (int mr = row_lo + et / tpr; mr < rows_valid; mr += 2 * rpp) {
          const int mr1 = mr + rpp;
          const bool has1 = mr1 < rows_valid;
          // residual first: an independent load whose latency then runs under the partial tiles'
          const bool pre = vec_ok && p.residual;
          uint4 rv0 = make_uint4(0, 0, 0, 0), rv1 = rv0;
          if (pre) {
            rv0 = __ldg(reinterpret_cast<const uint4*>(p.residual + (size_t)(m0 + mr) * p.ldo + n_out0));
            if (has1) rv1 = __ldg(reinterpret_cast<const uint4*>(p.residual + (size_t)(m0 + mr1) * p.ldo + n_out0));
          }
          float x0[16], x1[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) { x0[i] = 0.f; x1[i] = 0.f; }
          for (int s0 = 0; s0 < nsrc; s0 += kMaxBatch) {
            float4 f0[kMaxBatch][4], f1[kMaxBatch][4];
#pragma unroll
            for (int sb = 0; sb < kMaxBatch; ++sb) {
              const bool on = s0 + sb < nsrc;
              const float* base = src + (size_t)(on ? s0 + sb : 0) * (TN * kTileN) + col0;
              const bool dsm = p.cluster && !p.cluster_ws;
              const uint32_t peer = dsm ? mb::dsmem_addr(mb::smem_u32(s_tile + col0), on ? s0 + sb : 0) : 0u;
#pragma unroll
              for (int i4 = 0; i4 < 4; ++i4) {
                const bool ld = on && i4 < nf4;
                const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
                if (dsm) {
                  f0[sb][i4] = ld ? mb::dsmem_ld_f4(peer + (mr * kTileN + i4 * 4) * 4) : z4;
                  f1[sb][i4] = (ld && has1) ? mb::dsmem_ld_f4(peer + (mr1 * kTileN + i4 * 4) * 4) : z4;
                } else {
                  f0[sb][i4] = ld ? __ldcg(reinterpret_cast<const float4*>(base + mr * kTileN) + i4) : z4;
                  f1[sb][i4] = (ld && has1) ? __ldcg(reinterpret_cast<const float4*>(base + mr1 * kTileN) + i4) : z4;
                }
              }
            }
#pragma unroll
            for (int sb = 0; sb < kMaxBatch; ++sb)
#pragma unroll
              for (int i4 = 0; i4 < 4; ++i4) {
                x0[i4 * 4] += f0[sb][i4].x; x0[i4 * 4 + 1] += f0[sb][i4].y;
                x0[i4 * 4 + 2] += f0[sb][i4].z; x0[i4 * 4 + 3] += f0[sb][i4].w;
                x1[i4 * 4] += f1[sb][i4].x; x1[i4 * 4 + 1] += f1[sb][i4].y;
                x1[i4 * 4 + 2] += f1[sb][i4].z; x1[i4 * 4 + 3] += f1[sb][i4].w;
              }
          }
          if (threadIdx.x == 64 && mr == row_lo) MB_STAMP(11);
          emit(mr, x0, pre ? &rv0 : nullptr);
          if (has1) emit(mr1, x1, pre ? &rv1 : nullptr);
        }
      }
    }
    if (threadIdx.x == 64 && p.cluster) MB_STAMP(10);
    if (p.splits > 1 && p.cluster && !p.cluster_ws) mb::cluster_sync_all();   // peers may still be reading this CTA's tile
    if (threadIdx.x == 64) MB_STAMP(6);
    mb::tc_fence_before();
  }
  __syncthreads();
  if (threadIdx.x == 0) MB_STAMP(7);
  if (warp == 1) {
    mb::tc_fence_after();
    mb::tmem_dealloc(tmem, C::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------
// Persistent variant for layers with more weight-row tiles than SMs (gate_up, lm_head) and one
// token tile (M <= 128): every CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... with the
// stage ring running across tile boundaries and two TMEM accumulators, so the epilogue of tile i
// (TMEM -> registers -> global, no shared-memory staging) overlaps the main loop of tile i + 1
// and the weight stream never pauses. Same operand kinds except the 128x128-block fp8 kind.
template <int KIND, int TN>
struct PCfg {
  static constexpr int kABytes = kTileN * 128;
  static constexpr int kBBytes = TN * 128;
  static constexpr int kSfBytes = (KIND == KIND_NVFP4) ? 2048 : 0;
  static constexpr int kStageBytes = kABytes + kBBytes + 2 * kSfBytes;
  static constexpr int kStagesRaw = (200 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSfBase = 2 * TN;                                        // after the two accumulators
  static constexpr int kNeedCols = 2 * TN + (KIND == KIND_NVFP4 ? 64 : 0);
  static constexpr int kTmemCols =
      kNeedCols <= 32 ? 32 : kNeedCols <= 64 ? 64 : kNeedCols <= 128 ? 128 : kNeedCols <= 256 ? 256 : 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
};

constexpr int kPersistThreads = 576;   // producer warp + MMA warp + 16 epilogue warps
constexpr int kEpiGroups = (kPersistThreads - 64) / 128;   // warps per TMEM lane quadrant

template <int KIND, int TN>
__global__ void __launch_bounds__(kPersistThreads, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const GemmParams p) {
  static_assert(KIND != KIND_FP8_BLOCK && TN <= 128, "unsupported persistent configuration");
  using C = PCfg<KIND, TN>;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) float s_ascale[2][TN];

  const int warp = threadIdx.x >> 5;
  const int n_tiles = (p.N + kTileN - 1) / kTileN;
  const int m_tiles = (p.M + TN - 1) / TN;               // 1 for decode; prefill walks token tiles fastest
  const int nkb = p.num_kb;
  // work item t = blockIdx.x + i * gridDim.x covers weight tile t / m_tiles and token tile t % m_tiles
  const int my_tiles = (n_tiles * m_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // grid <= tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mb::mbar_init(&full_bar[s], 1);
      mb::mbar_init(&empty_bar[s], 1);
    }
    mb::mbar_init(&acc_full[0], 1);
    mb::mbar_init(&acc_full[1], 1);
    mb::mbar_init(&acc_empty[0], kPersistThreads - 64);
    mb::mbar_init(&acc_empty[1], kPersistThreads - 64);
    mb::mbar_fence_init();
    mb::tma_prefetch_desc(&tmA);
    mb::tma_prefetch_desc(&tmB);
  }
  if (warp == 1) mb::tmem_alloc(&tmem_base_s, C::kTmemCols);
  mb::tc_fence_before();
  __syncthreads();
  mb::tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  mb::pdl_launch_dependents();

  auto sA = [&](int s) { return smem + s * C::kStageBytes; };
  auto sB = [&](int s) { return smem + s * C::kStageBytes + C::kABytes; };
  auto sSFA = [&](int s) { return smem + s * C::kStageBytes + C::kABytes + C::kBBytes; };
  auto sSFB = [&](int s) { return smem + s * C::kStageBytes + C::kABytes + C::kBBytes + C::kSfBytes; };
  constexpr int kCoordStep = (KIND == KIND_BF16) ? 64 : 128;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (mb::elect_one()) {
      const int total = my_tiles * nkb;                   // k blocks this CTA streams, over all its tiles
      // both streams are issued in increasing g: the (work item, k block) cursors advance
      // incrementally, with one division per work item instead of several per k block
      int w_kb = 0, w_item = (int)blockIdx.x, w_tile = w_item / m_tiles;
      auto load_w = [&](int g) {
        const int s = g % kStages;
        mb::tma_load_2d(sA(s), &tmA, &full_bar[s], w_kb * kCoordStep, w_tile * kTileN);
        if constexpr (KIND == KIND_NVFP4)
          mb::bulk_load(sSFA(s), p.sfa + ((size_t)w_tile * p.sf_k64 + (size_t)w_kb * 4) * 512, 2048, &full_bar[s]);
        if (++w_kb == nkb) { w_kb = 0; w_item += (int)gridDim.x; w_tile = w_item / m_tiles; }
      };
      int x_kb = 0, x_item = (int)blockIdx.x, x_mt = x_item % m_tiles;
      auto load_x = [&](int g) {
        const int s = g % kStages;
        mb::tma_load_2d(sB(s), &tmB, &full_bar[s], x_kb * kCoordStep, x_mt * TN);
        if constexpr (KIND == KIND_NVFP4)
          mb::bulk_load(sSFB(s), p.sfb + ((size_t)((x_mt * TN) / 128) * p.sf_k64 + (size_t)x_kb * 4) * 512, 2048, &full_bar[s]);
        if (++x_kb == nkb) { x_kb = 0; x_item += (int)gridDim.x; x_mt = x_item % m_tiles; }
      };
      const int pre = min(total, kStages);
      for (int g = 0; g < pre; ++g) {                     // weights do not depend on the preceding kernel
        mb::mbar_expect_tx(&full_bar[g], C::kStageBytes);
        load_w(g);
      }
      mb::pdl_wait();
      for (int g = 0; g < pre; ++g) load_x(g);
      const bool skip_x = MB_DBG(32);                     // timing experiments: stale activation tiles
      for (int g = pre; g < total; ++g) {
        const int s = g % kStages;
        const uint32_t ph = (g / kStages) & 1;
        if (!mb::mbar_wait(&empty_bar[s], ph ^ 1, p.status, MB_ST_TIMEOUT_TMA)) break;
        mb::mbar_expect_tx(&full_bar[s], C::kStageBytes - (skip_x ? C::kBBytes + C::kSfBytes : 0));
        load_w(g);
        if (!skip_x) load_x(g);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (mb::elect_one()) {
      uint32_t idesc;
      if constexpr (KIND == KIND_BF16) idesc = mb::umma_idesc(1, 1, kTileN, TN);
      else if constexpr (KIND == KIND_NVFP4) idesc = mb::umma_idesc_bs(1, 1, kTileN, TN, 0);
      else idesc = mb::umma_idesc(0, 0, kTileN, TN);
      bool ok = true;
      int g = 0;
      for (int it = 0; it < my_tiles && ok; ++it) {
        const int buf = it & 1;
        // the epilogue must have drained this accumulator (two tiles ago) before it is overwritten
        ok = mb::mbar_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1, p.status, MB_ST_TIMEOUT_MMA);
        if (!ok) break;
        mb::tc_fence_after();
        const uint32_t acc = tmem + buf * TN;
        for (int i = 0; i < nkb; ++i, ++g) {
          const int s = g % kStages;
          const uint32_t ph = (g / kStages) & 1;
          ok = mb::mbar_wait(&full_bar[s], ph, p.status, MB_ST_TIMEOUT_MMA);
          if (!ok) break;
          mb::tc_fence_after();
          const uint32_t a_base = mb::smem_u32(sA(s)), b_base = mb::smem_u32(sB(s));
          const uint32_t sfa_col = C::kSfBase + (g & 1) * 32, sfb_col = sfa_col + 16;
          if constexpr (KIND == KIND_NVFP4) {
            const uint32_t sfa = mb::smem_u32(sSFA(s)), sfb = mb::smem_u32(sSFB(s));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              mb::tmem_cp_sf(tmem + sfa_col + j * 4, mb::umma_desc_sf(sfa + j * 512));
              mb::tmem_cp_sf(tmem + sfb_col + j * 4, mb::umma_desc_sf(sfb + j * 512));
            }
          }
          if (!MB_DBG(4)) {                             // timing experiments: no MMAs
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t da = mb::umma_desc_sw128(a_base + j * 32);
            const uint64_t db = mb::umma_desc_sw128(b_base + j * 32);
            if constexpr (KIND == KIND_BF16) mb::umma_f16(acc, da, db, idesc, (i | j) != 0);
            else if constexpr (KIND == KIND_FP8) mb::umma_f8f6f4(acc, da, db, idesc, (i | j) != 0);
            else mb::umma_nvfp4(acc, da, db, idesc, tmem + sfa_col + j * 4, tmem + sfb_col + j * 4, (i | j) != 0);
          }
          }
          mb::tc_commit(&empty_bar[s]);
        }
        if (ok) mb::tc_commit(&acc_full[buf]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue: TMEM -> registers -> global
    // kEpiGroups warps per TMEM lane quadrant (a warp may only read the quadrant warp_id % 4),
    // each taking every kEpiGroups-th 16-token chunk, which shortens the exposed epilogue of a
    // CTA's last tile accordingly
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int lane = threadIdx.x & 31;
    const int et = threadIdx.x - 64;
    const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
    const bool swiglu = p.epilogue == EPI_SWIGLU;
    mb::pdl_wait();
    const int f = q * 32 + lane;                          // weight row of this thread inside a tile
    const float outq_inv6gs = p.outq ? 1.f / (6.f * p.outq_gs) : 0.f;
    bool ok = true;
    for (int it = 0; it < my_tiles && ok; ++it) {
      const int t_lin = (int)blockIdx.x + it * (int)gridDim.x;
      const int tile = t_lin / m_tiles;
      const int m_base = (t_lin % m_tiles) * TN;           // first token row of this tile
      const int m_valid = min(p.M - m_base, TN);
      const int buf = it & 1;
      if (it == 0 || m_tiles > 1) {
        // per-token activation scales of this token tile. Two buffers and one barrier per tile:
        // nobody can be two tiles ahead of a thread that has not passed the barrier in between.
        for (int j = et; j < TN; j += kPersistThreads - 64) {
          float sc = 1.f;
          if constexpr (KIND == KIND_FP8 || KIND == KIND_NVFP4) {
            if (p.a_scale && j < m_valid) sc = __ldg(&p.a_scale[m_base + j]);
          }
          s_ascale[buf][j] = sc;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kPersistThreads - 64) : "memory");
      }
      const float* asc = s_ascale[m_tiles > 1 ? buf : 0];
      ok = mb::mbar_wait(&acc_full[buf], (it >> 1) & 1, p.status, MB_ST_TIMEOUT_EPI);
      if (!ok) break;
      mb::tc_fence_after();
      const int n = tile * kTileN + f;
      float wsc = p.alpha;
      if constexpr (KIND == KIND_FP8 || KIND == KIND_NVFP4) {
        if (p.w_scale && n < p.N) wsc *= __ldg(&p.w_scale[n]);
      }
      for (int c = half; c * 16 < m_valid && !MB_DBG(2); c += kEpiGroups) {   // dbg 2: timing experiments, no epilogue
        float v[16];
        mb::tmem_ld16(lane_addr + buf * TN + c * 16, v);
        if (swiglu) {
          // rows are interleaved (gate, up): an even lane holds the gate row, its odd neighbour
          // the up row. Per pair of tokens the even lane finishes token j, the odd one token
          // j + 1 (branch-free: both lanes run the same instruction stream).
          const bool odd = lane & 1;
          const bool n_ok = odd ? (n < p.N) : (n + 1 < p.N);
          __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(p.out) + (n >> 1);
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const int m0 = c * 16 + j;
            const float2 as = *reinterpret_cast<const float2*>(&asc[m0]);
            const float x0 = v[j] * (wsc * as.x), x1 = v[j + 1] * (wsc * as.y);
            const float other = __shfl_xor_sync(0xffffffffu, odd ? x0 : x1, 1);
            const float gate = odd ? other : x0, up = odd ? x1 : other;
            const float y = mb::silu(gate) * up;
            const int ml = m0 + (odd ? 1 : 0);                 // row inside the tile
            const int m = m_base + ml;
            if (p.outq) {
              // This warp's 16 even lanes hold one 16-wide quantisation block of token m0, its odd
              // lanes the same block of token m0 + 1 (block index along the consumer's K: tile * 4 + q).
              const float yv = n_ok ? y : 0.f;
              float bmax = fabsf(yv);
              bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 2));
              bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 4));
              bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 8));
              bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 16));
              const uint8_t sfc = mb::float_to_e4m3(bmax * outq_inv6gs);
              const float sff = mb::e4m3_to_float(sfc);
              const float qi = sff > 0.f ? __fdividef(1.f, sff * p.outq_gs) : 0.f;
              const float scaled = yv * qi;
              // outputs 2i and 2i + 1 of the block sit two lanes apart: the lower one packs the byte
              const float upper = __shfl_down_sync(0xffffffffu, scaled, 2);
              const uint32_t byte = mb::e2m1x2_pack(scaled, upper);
              const int i = lane >> 1;                      // output index inside the block
              if (ml < m_valid && !(i & 1) && n < p.N)
                p.outq[(size_t)m * p.ldq + ((tile * 64 + q * 16 + i) >> 1)] = (uint8_t)byte;
              if (ml < m_valid && i == 0 && n < p.N) {
                const int kb = tile * 4 + q;
                p.outq_sf[((size_t)(m >> 7) * p.outq_sf_k64 + (kb >> 2)) * 512 + mb::sf_tile_offset(m & 127, kb & 3)] = sfc;
              }
            } else if (n_ok && ml < m_valid) {
              outp[(size_t)m * p.ldo] = __float2bfloat16(y);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int ml = c * 16 + j;
            if (ml < m_valid && n < p.N) {
              float y = v[j] * wsc * asc[ml];
              const size_t o = (size_t)(m_base + ml) * p.ldo + n;
              if (p.residual) y += __bfloat162float(p.residual[o]);
              if (p.out_f32) reinterpret_cast<float*>(p.out)[o] = y;
              else reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16(y);
            }
          }
        }
      }
      mb::tc_fence_before();
      mb::mbar_arrive(&acc_empty[buf]);
    }
    mb::tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    mb::tc_fence_after();
    mb::tmem_dealloc(tmem, C::kTmemCols);
  }
}

template <int KIND, int TN>
int launch_persistent(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid_x,
                      cudaStream_t stream) {
  using C = PCfg<KIND, TN>;
  static bool configured = false;
  auto kern = gemm_persistent_kernel<KIND, TN>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)mb::launch_kernel_cluster(kern, dim3(grid_x), dim3(kPersistThreads), C::kSmemBytes, stream, 1, tmA, tmB, p);
}

template <int KIND>
int dispatch_persistent(int tn, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid_x,
                        cudaStream_t stream) {
  switch (tn) {
    case 16: return launch_persistent<KIND, 16>(tmA, tmB, p, grid_x, stream);
    case 32: return launch_persistent<KIND, 32>(tmA, tmB, p, grid_x, stream);
    case 64: return launch_persistent<KIND, 64>(tmA, tmB, p, grid_x, stream);
    case 128: return launch_persistent<KIND, 128>(tmA, tmB, p, grid_x, stream);
    default: return MB_ERR_UNSUPPORTED;
  }
}

template <int KIND, int TN, int CTAS = 1>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, dim3 grid,
           cudaStream_t stream) {
  const int cluster_z = p.cluster ? p.splits : 1;
  using C = Cfg<KIND, TN, CTAS>;
  static bool configured = false;
  auto kern = gemm_kernel<KIND, TN, CTAS>;
  if (!configured) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)mb::launch_kernel_cluster(kern, grid, dim3(192), C::kSmemBytes, stream, cluster_z, tmA, tmB, p);
}

template <int KIND>
int dispatch_tn(int tn, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                dim3 grid, cudaStream_t stream) {
  switch (tn) {
    case 16: return launch<KIND, 16>(tmA, tmB, p, grid, stream);
    case 32: return launch<KIND, 32>(tmA, tmB, p, grid, stream);
    case 64: return launch<KIND, 64>(tmA, tmB, p, grid, stream);
    case 128: return launch<KIND, 128>(tmA, tmB, p, grid, stream);
    default: break;
  }
  if constexpr (KIND == KIND_BF16 || KIND == KIND_FP8) {
    if (tn == 256) return launch<KIND, 256>(tmA, tmB, p, grid, stream);
  }
  return MB_ERR_UNSUPPORTED;
}

}  // namespace

extern "C" {

// Bytes of split-K workspace needed for (M, N, K, kind) under the default
// heuristics; the first `mb_gemm_counter_bytes` bytes of the workspace hold the
// per-tile arrival counters and must be zero before the first launch.
size_t mb_gemm_counter_bytes() { return 64 * 1024; }


int mb_gemm(const MbGemmArgs* a, cudaStream_t stream) {
  if (!a || !a->W || !a->X || !a->out || a->M <= 0 || a->N <= 0 || a->K <= 0) return MB_ERR_BAD_ARG;
  const int kind = a->kind;
  int kelems, elem_bits;
  CUtensorMapDataType dt;
  switch (kind) {
    case KIND_BF16: kelems = 64; elem_bits = 16; dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case KIND_FP8:
    case KIND_FP8_BLOCK: kelems = 128; elem_bits = 8; dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    case KIND_NVFP4: kelems = 256; elem_bits = 4; dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    default: return MB_ERR_UNSUPPORTED;
  }
  const size_t row_bytes = (size_t)a->K * elem_bits / 8;
  if (row_bytes % 16) return MB_ERR_BAD_ARG;           // TMA global stride rule
  if (kind == KIND_NVFP4 && (!a->sfa || !a->sfb)) return MB_ERR_BAD_ARG;
  if (kind == KIND_FP8_BLOCK && (!a->w_scale || !a->a_scale)) return MB_ERR_BAD_ARG;
  if (a->epilogue == EPI_SWIGLU && (a->out_f32 || a->residual)) return MB_ERR_BAD_ARG;
  const int num_kb = (a->K + kelems - 1) / kelems;
  if (kind == KIND_NVFP4 && a->sf_k64 < num_kb * 4) return MB_ERR_BAD_ARG;

  int tn = a->force_tn;
  const int tn_cap = (kind == KIND_BF16 || kind == KIND_FP8) ? 256 : 128;
  if (tn <= 0) {
    tn = 16;
    while (tn < a->M && tn < tn_cap) tn <<= 1;
  }
  if (kind == KIND_FP8_BLOCK && tn > 64) tn = 64;       // register-resident promotion
  const bool grouped = a->tile_expert != nullptr;
  if (grouped) {
    if (!a->tile_row0 || !a->tile_nrows || a->n_per_expert <= 0 || a->n_per_expert % kTileN ||
        a->max_tiles <= 0)
      return MB_ERR_UNSUPPORTED;
    // NVFP4 scale factors come in blocks of 128 rows: every tile of the work list must start at a multiple
    // of 128 rows (the sort lays the tiles out that way) and takes the first force_tn rows of its block
    if (kind == KIND_NVFP4) {
      if ((a->force_tn != 16 && a->force_tn != 32 && a->force_tn != 64 && a->force_tn != 128) || a->M % 128)
        return MB_ERR_UNSUPPORTED;
    } else if (tn > 64) {
      tn = 64;
    }
  }
  const int tiles_n = grouped ? a->n_per_expert / kTileN : (a->N + kTileN - 1) / kTileN;
  const int tiles_m = grouped ? a->max_tiles : (a->M + tn - 1) / tn;
  if (kind == KIND_FP8_BLOCK && !grouped && a->a_ld < tiles_m * tn) return MB_ERR_BAD_ARG;
  if (kind == KIND_FP8_BLOCK && grouped && a->a_ld < a->M + tn) return MB_ERR_BAD_ARG;
  // scale-factor tiles are 128 rows: several token tiles only line up at TN = 128
  if (kind == KIND_NVFP4 && !grouped && tiles_m > 1 && tn != 128) return MB_ERR_BAD_ARG;
  const int tiles = tiles_n * tiles_m;
  const int sms = a->sm_count > 0 ? a->sm_count : 148;
  int splits = a->force_splits;
  if (splits <= 0) {
    splits = 1;
    if (tiles < sms && a->ws) {
      splits = sms / tiles;
      const int max_by_k = num_kb / 4 > 0 ? num_kb / 4 : 1;
      if (splits > max_by_k) splits = max_by_k;
      if (splits < 1) splits = 1;
    }
  }
  if (splits > num_kb) splits = num_kb;
  int kb_per = (num_kb + splits - 1) / splits;
  splits = (num_kb + kb_per - 1) / kb_per;              // no empty split

  GemmParams p{};
  p.M = a->M; p.N = a->N; p.K = a->K; p.ldo = a->ldo;
  p.out = a->out;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a->residual);
  p.w_scale = a->w_scale; p.a_scale = a->a_scale; p.a_ld = a->a_ld;
  p.alpha = a->alpha;
  p.sfa = reinterpret_cast<const uint8_t*>(a->sfa);
  p.sfb = reinterpret_cast<const uint8_t*>(a->sfb);
  p.sf_k64 = a->sf_k64;
  p.splits = splits; p.kb_per_split = kb_per; p.num_kb = num_kb;
  p.epilogue = a->epilogue; p.out_f32 = a->out_f32;
  p.status = a->status;
#ifdef MB_GEMM_TIMING_EXPERIMENTS
  p.dbg = a->flags & 47;
  p.trace = a->timing_trace;
#endif
  p.tile_expert = a->tile_expert; p.tile_row0 = a->tile_row0; p.tile_nrows = a->tile_nrows;
  p.n_per_expert = grouped ? a->n_per_expert : 0;
  p.cluster = (splits > 1 && splits <= 8 && !a->no_cluster) ? 1 : 0;
  // exchange through the workspace when it is there and large enough (the fused tensor-parallel
  // epilogue keeps its tiles in shared memory)
  p.cluster_ws = (p.cluster && a->ws && !(a->flags & MB_GEMM_DSMEM_SPLITK) &&
                  a->ws_bytes >= mb_gemm_counter_bytes() + (size_t)tiles * splits * tn * kTileN * sizeof(float)) ? 1 : 0;
  if (a->outq) {
    if (a->epilogue != EPI_SWIGLU || !a->outq_sf || a->outq_gs <= 0.f || (a->N / 2) % 16 || a->outq_sf_k64 * 64 < a->N / 2)
      return MB_ERR_BAD_ARG;
    p.outq = reinterpret_cast<uint8_t*>(a->outq); p.ldq = a->ldq;
    p.outq_sf = reinterpret_cast<uint8_t*>(a->outq_sf); p.outq_sf_k64 = a->outq_sf_k64;
    p.outq_gs = a->outq_gs;
  }
  if (splits > 1 && (!p.cluster || p.cluster_ws)) {
    const size_t cbytes = mb_gemm_counter_bytes();
    const size_t need = cbytes + (size_t)tiles * splits * tn * kTileN * sizeof(float);
    if (!a->ws || a->ws_bytes < need || (!p.cluster && (size_t)tiles * 4 > cbytes)) return MB_ERR_TOO_LARGE;
    p.cnt = reinterpret_cast<uint32_t*>(a->ws);
    p.ws = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a->ws) + cbytes);
  }

  CUtensorMap tmA, tmB;
  const uint64_t inner = (uint64_t)row_bytes * 8 / (elem_bits == 4 ? 8 : elem_bits);
  const uint32_t box_inner = (elem_bits == 16) ? 64 : 128;
  int rc = mbh::encode_2d(&tmA, dt, a->W, inner, (uint64_t)a->N, row_bytes, box_inner, kTileN);
  if (rc) return rc;
  rc = mbh::encode_2d(&tmB, dt, a->X, inner, (uint64_t)a->M, row_bytes, box_inner, (uint32_t)tn);
  if (rc) return rc;

  // prefill-sized plain GEMMs put the token tiles in x (MB_GEMM_DECODE_TILE_ORDER keeps the decode order)
  p.m_fastest = (!grouped && tiles_m >= 8 && tiles_m <= 65535 && tiles_n <= 65535 && !(a->flags & MB_GEMM_DECODE_TILE_ORDER)) ? 1 : 0;
  dim3 grid(p.m_fastest ? tiles_m : tiles_n, p.m_fastest ? tiles_n : tiles_m, splits);
  rc = MB_ERR_UNSUPPORTED;
  // more tiles than SMs: persistent CTAs, balanced tile counts. One token tile (decode) always;
  // several token tiles (prefill, 128-token tiles) when MB_GEMM_PERSISTENT_PREFILL asks for it.
  const bool multi_m_ok = tiles_m > 1 && tn == 128 && (a->flags & MB_GEMM_PERSISTENT_PREFILL) && !a->outq;
  if (!grouped && splits == 1 && (tiles_m == 1 || multi_m_ok) && tn <= 128 && kind != KIND_FP8_BLOCK &&
      tiles > sms && (tiles_m > 1 || tiles_n > sms) && !(a->flags & MB_GEMM_ONE_TILE_PER_CTA)) {
    const int waves = (tiles + sms - 1) / sms;
    const int grid_x = (tiles + waves - 1) / waves;
    switch (kind) {
      case KIND_BF16: return dispatch_persistent<KIND_BF16>(tn, tmA, tmB, p, grid_x, stream);
      case KIND_FP8: return dispatch_persistent<KIND_FP8>(tn, tmA, tmB, p, grid_x, stream);
      default: return dispatch_persistent<KIND_NVFP4>(tn, tmA, tmB, p, grid_x, stream);
    }
  }
  if (a->outq) return MB_ERR_UNSUPPORTED;      // only the persistent epilogue quantises
  if (grouped && tn <= 32 && !(a->flags & MB_GEMM_GROUPED_ONE_CTA)) {
    // small token tiles of a MoE work list: two CTAs per SM with half the stages each
    const bool t16 = tn == 16;
    switch (kind) {
      case KIND_BF16: return t16 ? launch<KIND_BF16, 16, 2>(tmA, tmB, p, grid, stream) : launch<KIND_BF16, 32, 2>(tmA, tmB, p, grid, stream);
      case KIND_FP8: return t16 ? launch<KIND_FP8, 16, 2>(tmA, tmB, p, grid, stream) : launch<KIND_FP8, 32, 2>(tmA, tmB, p, grid, stream);
      case KIND_NVFP4: return t16 ? launch<KIND_NVFP4, 16, 2>(tmA, tmB, p, grid, stream) : launch<KIND_NVFP4, 32, 2>(tmA, tmB, p, grid, stream);
      default: return t16 ? launch<KIND_FP8_BLOCK, 16, 2>(tmA, tmB, p, grid, stream) : launch<KIND_FP8_BLOCK, 32, 2>(tmA, tmB, p, grid, stream);
    }
  }
  switch (kind) {
    case KIND_BF16: rc = dispatch_tn<KIND_BF16>(tn, tmA, tmB, p, grid, stream); break;
    case KIND_FP8: rc = dispatch_tn<KIND_FP8>(tn, tmA, tmB, p, grid, stream); break;
    case KIND_NVFP4: rc = dispatch_tn<KIND_NVFP4>(tn, tmA, tmB, p, grid, stream); break;
    case KIND_FP8_BLOCK:
      switch (tn) {
        case 16: rc = launch<KIND_FP8_BLOCK, 16>(tmA, tmB, p, grid, stream); break;
        case 32: rc = launch<KIND_FP8_BLOCK, 32>(tmA, tmB, p, grid, stream); break;
        case 64: rc = launch<KIND_FP8_BLOCK, 64>(tmA, tmB, p, grid, stream); break;
        default: rc = MB_ERR_UNSUPPORTED;
      }
      break;
  }
  return rc;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Allocation-free entry point (declared in noalloc.h).
//
// Some callers may not allocate device memory at all: code running between
// cudaStreamBeginCapture and cudaStreamEndCapture, plugins that live inside another
// framework's memory plan, and real-time loops that must not touch the allocator. The
// split-K GEMM normally gets its partial-tile workspace from the caller; this variant
// keeps that workspace in a file-scope device array instead, so the only pointers the
// caller supplies are operands and outputs.
//
// The array's name is only a host-side handle: the device address is obtained once per
// device with cudaGetSymbolAddress (with that device current) on the first call made on
// that device, which also zeroes the arrival counters. That first call should therefore be
// made before any stream capture starts. Every call on a device shares the one array and
// it keeps the previous call's partial tiles; the counters re-arm themselves, nothing else
// needs clearing. Two calls that overlap on the GPU (different streams) would race on the
// array: serialise them. Problem sizes whose workspace exceeds MB_NOALLOC_SCRATCH_BYTES are
// refused with MB_ERR_TOO_LARGE. No cudaMalloc / cudaFree / allocating library call is made.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MB_NOALLOC_SCRATCH_BYTES];

extern "C" int mb_gemm_noalloc(const MbGemmArgs* a, cudaStream_t stream) {
  if (!a) return MB_ERR_BAD_ARG;
  static void* dev_ptr[64] = {nullptr};
  static std::mutex setup_lock;          // first calls from several threads set a device up once
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return MB_ERR_UNSUPPORTED;
  {
    std::lock_guard<std::mutex> guard(setup_lock);
    if (!dev_ptr[dev]) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
      if (e != cudaSuccess) return (int)e;
      // arrival counters start at zero; the set-up call waits for this, so that a first pair of
      // calls on two different streams cannot see the second one run ahead of the clearing
      e = cudaMemsetAsync(ptr, 0, mb_gemm_counter_bytes(), stream);
      if (e != cudaSuccess) return (int)e;
      e = cudaStreamSynchronize(stream);
      if (e != cudaSuccess) return (int)e;
      dev_ptr[dev] = ptr;
    }
  }
  MbGemmArgs b = *a;
  b.ws = dev_ptr[dev];
  b.ws_bytes = MB_NOALLOC_SCRATCH_BYTES;
  b.no_cluster = 1;            // this variant is the workspace path by definition
  return mb_gemm(&b, stream);  // refuses with MB_ERR_TOO_LARGE when the workspace would not fit
}
