// Tensor-parallel communication over NVLink peer memory (one process per GPU, symmetric buffers).
//
// The reference has no communication backend at all: its "NcclCollectives" and tensor-parallel
// forward are CPU simulations over threads (crates/oxibonsai-model/src/multi_gpu.rs:159-238,
// tensor_parallel.rs:338-386).  Here every rank maps every peer's symmetric buffer and kernels
// exchange data with plain st.global / ld.global to peer addresses plus release/acquire flags:
//
//   * fused row-parallel GEMV -> all-reduce + residual (one-shot, push based), two protocols:
//     flag-in-data (bitgemv_stream.cu): every finished row goes to slot [my rank] of every peer as
//     one 8-byte {value, tag} store and the receiving thread polls the payload itself, so there is
//     no fence and no separate flag round trip; tile flags (bitgemv.cu, the exact-f32 path): rows
//     first, then an epoch flag per (rank, tile) behind a system fence.  Either way the slots are
//     summed in rank order - every rank computes bit-identical hidden states;
//   * logits all-gather for the vocab-parallel LM head, and a two-shot in-place all-reduce for
//     the prefill GEMM outputs, both bracketed by flag barriers.
//
// No TMA load, bulk copy or library call ever takes a peer address: remote data moves only
// through ordinary loads and stores issued by these kernels.  Every wait is bounded; on expiry
// the kernel records an error code in *status and carries on without the missing data, so a
// rank that dies between steps cannot hang its peers' GPUs.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace bonsai {

constexpr int kTpMaxRanks = 8;
constexpr int kTpMaxTiles = 4096;
constexpr uint32_t kTpDefaultSpinLimit = 1u << 22;   // x ~0.2 us per poll: about a second

// Offsets inside every rank's symmetric buffer.
struct TpLayout {
  size_t off_tile_flags;   // int [2][kTpMaxRanks][kTpMaxTiles]
  size_t off_bar_flags;    // int [kTpMaxRanks]
  size_t off_recv;         // float [2][kTpMaxRanks][recv_elems]
  size_t off_logits;       // float [max_batch][vocab]
  size_t off_big;          // float [big_elems]  (prefill partial sums)
  size_t off_ll;           // u64 [2][kTpMaxRanks][recv_elems]  ({value, tag} slots of the flag-in-data exchange, one token)
  size_t off_ll_big;       // u64 [2][kTpMaxRanks][ll_big_elems]  (the same for decode batches: [token][row])
  size_t recv_elems, big_elems, ll_big_elems, total_bytes;
};

struct TpComm {
  int rank, size;
  uint8_t* peer[kTpMaxRanks];   // peer[r] = rank r's symmetric buffer as mapped in this process
  TpLayout lay;
  int* epoch;      // device int: number of fused all-reduces completed (local memory)
  int* done_ctr;   // device int: CTAs finished in the running fused kernel
  int* bar_epoch;  // device int: number of flag barriers completed
  int* status;     // device int: non-zero after a bounded wait expired
  uint32_t spin_limit;   // polls before a wait on a peer gives up (host-settable; tests use a small value)
  // Multicast mapping of the symmetric buffer (same layout; null when the fabric offers none or the path is switched
  // off): a multimem store through it lands in every rank's buffer, a multimem load-reduce returns the sum over all
  // ranks' buffers, both done by the NVLink switch.
  uint8_t* mc;
};

__device__ __forceinline__ void st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_volatile(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait until *flag >= want (epochs only grow).  Returns false on expiry.
__device__ __forceinline__ bool tp_wait_flag(const int* flag, int want, uint32_t spin_limit) {
  for (uint32_t i = 0; i < spin_limit; ++i) {
    if (ld_acquire_sys(flag) - want >= 0) return true;
    __nanosleep(20);
  }
  return false;
}

__device__ __forceinline__ float* tp_recv_slot(const TpComm& c, int on_rank, int parity, int from_rank) {
  return reinterpret_cast<float*>(c.peer[on_rank] + c.lay.off_recv) + ((size_t)parity * kTpMaxRanks + from_rank) * c.lay.recv_elems;
}
__device__ __forceinline__ unsigned long long* tp_ll_slot(const TpComm& c, int on_rank, int parity, int from_rank) {
  return reinterpret_cast<unsigned long long*>(c.peer[on_rank] + c.lay.off_ll) + ((size_t)parity * kTpMaxRanks + from_rank) * c.lay.recv_elems;
}
__device__ __forceinline__ unsigned long long* tp_ll_big_slot(const TpComm& c, int on_rank, int parity, int from_rank) {
  return reinterpret_cast<unsigned long long*>(c.peer[on_rank] + c.lay.off_ll_big) + ((size_t)parity * kTpMaxRanks + from_rank) * c.lay.ll_big_elems;
}
__device__ __forceinline__ void tp_st_msg(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// One {value, tag} message to the same slot of every rank's buffer (mc_slot: the slot's address in the multicast mapping).
__device__ __forceinline__ void tp_mc_st_msg(unsigned long long* mc_slot, unsigned long long v) {
  asm volatile("multimem.st.relaxed.sys.global.b64 [%0], %1;" ::"l"(mc_slot), "l"(v) : "memory");
}
__device__ __forceinline__ void tp_mc_st_f32(float* mc_p, float v) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc_p), "f"(v) : "memory");
}
__device__ __forceinline__ void tp_mc_st_f4(float4* mc_p, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// Sum over all ranks of the float4 at this offset of their buffers, added inside the switch.
__device__ __forceinline__ float4 tp_mc_ld_reduce_f4(const float4* mc_p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc_p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long* tp_ll_slot_mc(const TpComm& c, int parity, int from_rank) {
  return reinterpret_cast<unsigned long long*>(c.mc + c.lay.off_ll) + ((size_t)parity * kTpMaxRanks + from_rank) * c.lay.recv_elems;
}
__device__ __forceinline__ unsigned long long* tp_ll_big_slot_mc(const TpComm& c, int parity, int from_rank) {
  return reinterpret_cast<unsigned long long*>(c.mc + c.lay.off_ll_big) + ((size_t)parity * kTpMaxRanks + from_rank) * c.lay.ll_big_elems;
}
__device__ __forceinline__ unsigned long long tp_ld_msg(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Polls a {value, tag} slot until the tag shows up.  `alive` goes false on expiry, after which later calls of the
// thread poll only once (a silent peer costs one wait limit per thread, not one per value).
__device__ __forceinline__ float tp_recv_msg(const TpComm& c, const unsigned long long* slot, uint32_t tag, bool& alive) {
  const uint32_t limit = alive ? c.spin_limit : 1u;
  for (uint32_t it = 0; it < limit; ++it) {
    const unsigned long long m = tp_ld_msg(slot);
    if ((uint32_t)(m >> 32) == tag) return __uint_as_float((uint32_t)m);
  }
  alive = false;
  atomicExch(c.status, 2);
  return 0.0f;
}
// The same for all peers at once: acc + sum over ranks (in rank order) of their value for this element, `own` being this
// rank's.  slot_of(r) is the address of rank r's {value, tag} slot in this rank's buffer.  Every round requests all
// outstanding slots before it looks at any of them, so the round trips to L2 overlap instead of queueing up behind one
// another (seven peers: one latency per round, not seven); the values are added only when all have arrived, in rank
// order, so every rank adds the same numbers in the same order.
template <class SlotFn>
__device__ __forceinline__ float tp_recv_sum(const TpComm& c, SlotFn slot_of, uint32_t tag, float own, float acc, bool& alive) {
  unsigned long long m[kTpMaxRanks];
  uint32_t pending = ((1u << c.size) - 1u) & ~(1u << c.rank);
  const uint32_t limit = alive ? c.spin_limit : 1u;
  for (uint32_t it = 0; it < limit && pending != 0u; ++it) {
#pragma unroll
    for (int r = 0; r < kTpMaxRanks; ++r)
      if ((pending >> r) & 1u) m[r] = tp_ld_msg(slot_of(r));
#pragma unroll
    for (int r = 0; r < kTpMaxRanks; ++r)
      if (((pending >> r) & 1u) && (uint32_t)(m[r] >> 32) == tag) pending &= ~(1u << r);
  }
  if (pending != 0u) {
    alive = false;
    atomicExch(c.status, 2);
  }
#pragma unroll
  for (int r = 0; r < kTpMaxRanks; ++r)
    if (r < c.size) acc += r == c.rank ? own : (((pending >> r) & 1u) ? 0.0f : __uint_as_float((uint32_t)m[r]));
  return acc;
}
__device__ __forceinline__ int* tp_tile_flag(const TpComm& c, int on_rank, int parity, int from_rank, int tile) {
  return reinterpret_cast<int*>(c.peer[on_rank] + c.lay.off_tile_flags) + ((size_t)parity * kTpMaxRanks + from_rank) * kTpMaxTiles + tile;
}

// Second half of the fused epilogue, called by all threads of the CTA after the tile's rows have
// been stored to every peer's slot [c.rank] (rows row0 .. row0+nrows-1, element offset elem0 + row):
// publish the tile, wait for the peers' copies of it, then h[row] = residual[row] + sum_r slot[r][row].
__device__ __forceinline__ void tp_tile_allreduce(const TpComm& c, int epoch, int tile, int row0, int nrows, int n_total,
                                                  size_t elem0, const float* residual, float* out) {
  const int parity = epoch & 1, want = epoch + 1;
  __syncthreads();
  if (threadIdx.x == 0) __threadfence_system();
  __syncthreads();
  if (threadIdx.x < c.size) {
    st_release_sys(tp_tile_flag(c, threadIdx.x, parity, c.rank, tile), want);
    if (!tp_wait_flag(tp_tile_flag(c, c.rank, parity, threadIdx.x, tile), want, c.spin_limit)) atomicExch(c.status, 2);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nrows; i += blockDim.x) {
    const int row = row0 + i;
    if (row >= n_total) break;
    float v = residual ? residual[row] : 0.0f;
    for (int r = 0; r < c.size; ++r) v += __ldcg(tp_recv_slot(c, c.rank, parity, r) + elem0 + row);
    out[row] = v;
  }
}

// Last CTA of the fused kernel bumps the epoch (every CTA has read it by then).
__device__ __forceinline__ void tp_finish_kernel(const TpComm& c, int epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    int prev = atomicAdd(c.done_ctr, 1);
    if (prev == (int)gridDim.x - 1) {
      *c.done_ctr = 0;
      *c.epoch = epoch + 1;
      __threadfence();
    }
  }
}

}  // namespace bonsai
