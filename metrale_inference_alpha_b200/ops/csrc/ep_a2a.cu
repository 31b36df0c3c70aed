// Expert-parallel all-to-all over NVLink peer memory (no NCCL on the data path).
//
// Every rank owns a landing zone [source rank][capacity][row bytes] in symmetric memory. A rank
// scatters rows straight into the owners' zones with 16-byte peer stores (dispatch: token rows to
// the ranks that hold their experts; return: expert outputs back to the token's rank, into the slot
// the token was sent from), publishes how many rows it sent, and raises a per-source flag with
// system-scope release; the receiver waits (bounded) for every source's flag with acquire loads.
// Flags carry a sequence number, landing zones are double-buffered by its parity, so a step never
// overwrites rows a slower peer is still reading and nothing needs resetting between steps.
// One 32-bit word of metadata travels with every row (the expert id on dispatch).
//
// The reference reaches expert parallelism with masked-local experts + an all-reduce of
// [tokens, hidden] (crates/model-layers/src/layers/moe/forward/ep_reduce.rs:21-52) and carries a
// dead token-dispatch table (layers/ep_dispatch.rs:3-9); this is the dispatch it does not have.
#include "common.cuh"

namespace {

struct A2aParams {
  const uint8_t* rows;         // [n, row_bytes] rows to send
  long long row_ld;            // bytes between rows
  int n, row_bytes;
  const int* dst_rank;         // [n] destination rank or -1 (row not sent)
  const int* dst_slot;         // [n] slot inside this rank's region of the destination zone
  const int* meta;             // [n] word delivered with the row, or null
  const int* send_count;       // [world] rows sent to each rank (device)
  int world, rank, capacity;
  uint8_t* zone[8];            // per destination rank: base of its landing zone for this parity
  int* zone_meta[8];           // per destination rank: [world][capacity] metadata, or null
  int* zone_count[8];          // per destination rank: [world] rows received from each source
  uint32_t* flag[8];           // per destination rank: [world] sequence numbers
  uint32_t seq;
  const uint32_t* seq_ptr;     // when set, the sequence number is read from device memory at run time
                               // (a replayed CUDA graph then sees the counter of the current step)
  uint32_t* done;              // local: CTA completion counter (self-resetting)
  uint32_t* status;
};

// grid (n rows), 128 threads
__global__ void a2a_scatter_kernel(const A2aParams p) {
  const int i = blockIdx.x;
  mb::pdl_wait();
  mb::pdl_launch_dependents();
  const int r = p.dst_rank[i];
  if (r >= 0) {
    const int slot = p.dst_slot[i];
    if (r >= p.world || slot < 0 || slot >= p.capacity) {
      if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0u, MB_ST_BOUNDS);
    } else {
      const uint4* src = reinterpret_cast<const uint4*>(p.rows + (size_t)i * p.row_ld);
      uint4* dst = reinterpret_cast<uint4*>(p.zone[r] + ((size_t)p.rank * p.capacity + slot) * p.row_bytes);
      for (int k = threadIdx.x; k < p.row_bytes / 16; k += blockDim.x) dst[k] = src[k];
      if (p.meta && threadIdx.x == 0) p.zone_meta[r][(size_t)p.rank * p.capacity + slot] = p.meta[i];
    }
  }
  // the last CTA to finish publishes the counts and raises this rank's flag on every peer
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(p.done, 1u);
    s_last = prev == gridDim.x - 1;
    if (s_last) *p.done = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (threadIdx.x < p.world) {
    const int d = threadIdx.x;
    p.zone_count[d][p.rank] = p.send_count[d];
    __threadfence_system();
    const uint32_t seq = p.seq_ptr ? *reinterpret_cast<const volatile uint32_t*>(p.seq_ptr) : p.seq;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flag[d] + p.rank), "r"(seq) : "memory");
  }
}

// one CTA: thread s waits (bounded) until source s has raised its flag to `seq`
__global__ void a2a_wait_kernel(const uint32_t* flags, int world, uint32_t seq, const uint32_t* seq_ptr,
                                uint32_t* status) {
  mb::pdl_wait();
  if ((int)threadIdx.x >= world) return;
  if (seq_ptr) seq = *reinterpret_cast<const volatile uint32_t*>(seq_ptr);
  const uint32_t* f = flags + threadIdx.x;
  const long long t0 = clock64();
  while (mb::ld_acquire_sys(f) != seq) {
    if (clock64() - t0 > (long long)MB_WAIT_CYCLES) {
      if (status) atomicCAS(status, 0u, MB_ST_TIMEOUT_PEER);
      return;
    }
    __nanosleep(64);
  }
}

}  // namespace

extern "C" {

struct MbA2aArgs {
  const void* rows;
  long long row_ld;
  int n, row_bytes;
  const int* dst_rank;
  const int* dst_slot;
  const int* meta;
  const int* send_count;
  int world, rank, capacity;
  void* zone[8];
  void* zone_meta[8];
  void* zone_count[8];
  void* flag[8];
  unsigned int seq;
  void* done;
  void* status;
  const void* seq_ptr;   // optional device-resident sequence number (overrides `seq`)
};

int mb_a2a_scatter(const MbA2aArgs* a, cudaStream_t stream) {
  if (!a || !a->rows || !a->dst_rank || !a->dst_slot || !a->send_count || !a->done || a->n <= 0) return MB_ERR_BAD_ARG;
  if (a->world < 1 || a->world > 8 || a->rank < 0 || a->rank >= a->world || a->row_bytes % 16 || a->row_ld % 16)
    return MB_ERR_BAD_ARG;
  A2aParams p{};
  p.rows = reinterpret_cast<const uint8_t*>(a->rows); p.row_ld = a->row_ld; p.n = a->n; p.row_bytes = a->row_bytes;
  p.dst_rank = a->dst_rank; p.dst_slot = a->dst_slot; p.meta = a->meta; p.send_count = a->send_count;
  p.world = a->world; p.rank = a->rank; p.capacity = a->capacity;
  for (int r = 0; r < a->world; ++r) {
    if (!a->zone[r] || !a->zone_count[r] || !a->flag[r] || (a->meta && !a->zone_meta[r])) return MB_ERR_BAD_ARG;
    p.zone[r] = reinterpret_cast<uint8_t*>(a->zone[r]);
    p.zone_meta[r] = reinterpret_cast<int*>(a->zone_meta[r]);
    p.zone_count[r] = reinterpret_cast<int*>(a->zone_count[r]);
    p.flag[r] = reinterpret_cast<uint32_t*>(a->flag[r]);
  }
  p.seq = a->seq;
  p.seq_ptr = reinterpret_cast<const uint32_t*>(a->seq_ptr);
  p.done = reinterpret_cast<uint32_t*>(a->done);
  p.status = reinterpret_cast<uint32_t*>(a->status);
  return (int)mb::launch_kernel(a2a_scatter_kernel, dim3(a->n), dim3(128), (size_t)0, stream, p);
}

int mb_a2a_wait(const void* flags, int world, unsigned int seq, void* status, cudaStream_t stream) {
  if (!flags || world < 1 || world > 8) return MB_ERR_BAD_ARG;
  return (int)mb::launch_kernel(a2a_wait_kernel, dim3(1), dim3(32), (size_t)0, stream,
                                reinterpret_cast<const uint32_t*>(flags), world, (uint32_t)seq,
                                static_cast<const uint32_t*>(nullptr), reinterpret_cast<uint32_t*>(status));
}

// same wait with the sequence number read from device memory (graph-capturable)
int mb_a2a_wait_dev(const void* flags, int world, const void* seq_ptr, void* status, cudaStream_t stream) {
  if (!flags || !seq_ptr || world < 1 || world > 8) return MB_ERR_BAD_ARG;
  return (int)mb::launch_kernel(a2a_wait_kernel, dim3(1), dim3(32), (size_t)0, stream,
                                reinterpret_cast<const uint32_t*>(flags), world, 0u,
                                reinterpret_cast<const uint32_t*>(seq_ptr), reinterpret_cast<uint32_t*>(status));
}

}  // extern "C"
