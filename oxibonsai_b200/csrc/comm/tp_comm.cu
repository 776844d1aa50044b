// Host API and stand-alone kernels of the tensor-parallel communicator (see tp_comm.cuh).
#include "tp_comm.cuh"

#include <cstring>

#include "../cuda/common.cuh"

namespace bonsai {

// Flag barrier across ranks (one CTA): tell every peer "rank c.rank reached barrier #e", then wait
// until every peer has said the same.  Data written to peers before the barrier is visible to
// them after it.
__global__ void tp_barrier_kernel(TpComm c) {
  __shared__ int s_e;
  if (threadIdx.x == 0) s_e = ld_volatile(c.bar_epoch);
  __syncthreads();
  const int want = s_e + 1;
  if (threadIdx.x < c.size) {
    __threadfence_system();
    int* theirs = reinterpret_cast<int*>(c.peer[threadIdx.x] + c.lay.off_bar_flags) + c.rank;
    st_release_sys(theirs, want);
    const int* mine = reinterpret_cast<const int*>(c.peer[c.rank] + c.lay.off_bar_flags) + threadIdx.x;
    if (!tp_wait_flag(mine, want, c.spin_limit)) atomicExch(c.status, 3);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *c.bar_epoch = want;
    __threadfence();
  }
}

// Vocab-parallel LM head: copy this rank's logits slice [batch][rows] into every rank's full
// logits area at column row0.
__global__ void tp_push_logits_kernel(TpComm c, const float* __restrict__ local, int slot0, int batch, int rows, int row0, int vocab) {
  const size_t total = (size_t)batch * rows;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int b = slot0 + (int)(i / rows), r = (int)(i % rows);
    const float v = local[i];
    const size_t at = (size_t)b * vocab + row0 + r;
    if (c.mc != nullptr) {
      tp_mc_st_f32(reinterpret_cast<float*>(c.mc + c.lay.off_logits) + at, v);
    } else {
      for (int p = 0; p < c.size; ++p) reinterpret_cast<float*>(c.peer[p] + c.lay.off_logits)[at] = v;
    }
  }
}

// Two-shot all-reduce of the `big` area, in place: rank r sums elements [r*n/size, (r+1)*n/size)
// over all ranks (peer loads, rank order) and writes the result back into every rank's area.
// Must sit between two flag barriers.
__global__ void tp_reduce_broadcast_kernel(TpComm c, size_t n) {
  const size_t per = (n / 4 + c.size - 1) / c.size;   // float4 units per rank
  const size_t lo = (size_t)c.rank * per, hi = min(n / 4, lo + per);
  for (size_t i = lo + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < hi; i += (size_t)gridDim.x * blockDim.x) {
    if (c.mc != nullptr) {   // the switch adds the ranks' values and replicates the result
      float4* at = reinterpret_cast<float4*>(c.mc + c.lay.off_big) + i;
      tp_mc_st_f4(at, tp_mc_ld_reduce_f4(at));
      continue;
    }
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < c.size; ++p) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(c.peer[p] + c.lay.off_big) + i);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    for (int p = 0; p < c.size; ++p) reinterpret_cast<float4*>(c.peer[p] + c.lay.off_big)[i] = s;
  }
}

// One-shot all-reduce fused with the residual add, for small tensors (a decode batch): every rank has
// written its partial sums into its own big area at float4 offset off4.  One launch does the entry
// barrier (CTA 0 tells the peers, every CTA waits for all of them), then h += sum over ranks in rank
// order through peer loads, so all ranks hold bit-identical h.  There is no exit barrier: callers
// alternate between the two halves of the big area, and a rank can only reach its next write of a
// half after all peers have entered the all-reduce in between, i.e. finished reading that half.
__global__ void tp_allreduce_oneshot_add_kernel(TpComm c, float* __restrict__ h, size_t n4, size_t off4) {
  __shared__ int s_e;
  if (threadIdx.x == 0) s_e = ld_volatile(c.bar_epoch);
  __syncthreads();
  const int want = s_e + 1;
  if (threadIdx.x < c.size) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<int*>(c.peer[threadIdx.x] + c.lay.off_bar_flags) + c.rank, want);
    }
    const int* mine = reinterpret_cast<const int*>(c.peer[c.rank] + c.lay.off_bar_flags) + threadIdx.x;
    if (!tp_wait_flag(mine, want, c.spin_limit)) atomicExch(c.status, 4);
  }
  __syncthreads();
  float4* h4 = reinterpret_cast<float4*>(h);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    float4 s = h4[i];
    if (c.mc != nullptr) {
      const float4 v = tp_mc_ld_reduce_f4(reinterpret_cast<const float4*>(c.mc + c.lay.off_big) + off4 + i);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    } else {
      for (int p = 0; p < c.size; ++p) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(c.peer[p] + c.lay.off_big) + off4 + i);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    }
    h4[i] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int prev = atomicAdd(c.done_ctr, 1);
    if (prev == (int)gridDim.x - 1) {   // every CTA has read bar_epoch by now
      *c.done_ctr = 0;
      *c.bar_epoch = want;
      __threadfence();
    }
  }
}

__global__ void tp_add_kernel(float* __restrict__ h, const float* __restrict__ add, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) h[i] += add[i];
}

}  // namespace bonsai

extern "C" {

// Layout of the symmetric buffer for the given sizes; returns the number of bytes every rank must allocate.
// {value, tag} slots for decode batches: up to 64 tokens of recv_elems rows each.
size_t bonsai_tp_ll_big_elems(size_t recv_elems) { return 64 * recv_elems; }

size_t bonsai_tp_layout(size_t recv_elems, size_t logits_elems, size_t big_elems, size_t* offsets /*[7]*/) {
  using namespace bonsai;
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  size_t o = 0;
  offsets[0] = o; o = up(o + sizeof(int) * 2 * kTpMaxRanks * kTpMaxTiles);
  offsets[1] = o; o = up(o + sizeof(int) * kTpMaxRanks);
  offsets[2] = o; o = up(o + sizeof(float) * 2 * kTpMaxRanks * recv_elems);
  offsets[3] = o; o = up(o + sizeof(float) * logits_elems);
  offsets[4] = o; o = up(o + sizeof(float) * big_elems);
  offsets[5] = o; o = up(o + sizeof(unsigned long long) * 2 * kTpMaxRanks * recv_elems);
  offsets[6] = o; o = up(o + sizeof(unsigned long long) * 2 * kTpMaxRanks * bonsai_tp_ll_big_elems(recv_elems));
  return o;
}

// peer_ptrs[r] = address of rank r's symmetric buffer in this process.  state = 4 zeroed device ints
// (epoch, done counter, barrier epoch, status) in ordinary local memory.
void* bonsai_tp_create(int rank, int size, const uint64_t* peer_ptrs, size_t recv_elems, size_t logits_elems, size_t big_elems,
                       int* state) {
  using namespace bonsai;
  if (size < 1 || size > kTpMaxRanks || rank < 0 || rank >= size) return nullptr;
  TpComm* c = new TpComm();
  std::memset(c, 0, sizeof(TpComm));
  c->rank = rank;
  c->size = size;
  for (int r = 0; r < size; ++r) c->peer[r] = reinterpret_cast<uint8_t*>(peer_ptrs[r]);
  size_t off[7];
  c->lay.total_bytes = bonsai_tp_layout(recv_elems, logits_elems, big_elems, off);
  c->lay.off_tile_flags = off[0];
  c->lay.off_bar_flags = off[1];
  c->lay.off_recv = off[2];
  c->lay.off_logits = off[3];
  c->lay.off_big = off[4];
  c->lay.off_ll = off[5];
  c->lay.off_ll_big = off[6];
  c->lay.ll_big_elems = bonsai_tp_ll_big_elems(recv_elems);
  c->spin_limit = kTpDefaultSpinLimit;
  c->lay.recv_elems = recv_elems;
  c->lay.big_elems = big_elems;
  c->epoch = state;
  c->done_ctr = state + 1;
  c->bar_epoch = state + 2;
  c->status = state + 3;
  return c;
}
void bonsai_tp_destroy(void* c) { delete static_cast<bonsai::TpComm*>(c); }
// Redirects the status word (where expired waits are recorded) to another device int of the caller.
void bonsai_tp_set_status_ptr(void* c, int* status) { static_cast<bonsai::TpComm*>(c)->status = status; }
// Polls a wait on a peer may take before it gives up and records a status code (default: about a second).
void bonsai_tp_set_spin_limit(void* c, unsigned int polls) { static_cast<bonsai::TpComm*>(c)->spin_limit = polls < 1 ? 1 : polls; }

int bonsai_tp_barrier(void* comm, cudaStream_t stream) {
  bonsai::tp_barrier_kernel<<<1, 32, 0, stream>>>(*static_cast<bonsai::TpComm*>(comm));
  return bonsai::launch_status();
}

// Gathers [batch][rows] logits slices of all ranks into this rank's full logits area (and everyone else's).
// Once the flag barrier that follows the pushes has completed the area holds [batch][vocab]; its address is
// bonsai_tp_logits_ptr().
// `local` holds rows of logits slots slot0 .. slot0+batch-1.
int bonsai_tp_allgather_logits_at(void* comm, const float* local, int slot0, int batch, int rows, int row0, int vocab,
                                  cudaStream_t stream) {
  using namespace bonsai;
  TpComm& c = *static_cast<TpComm*>(comm);
  if (rows > 0) {
    int grid = (int)(((size_t)batch * rows + 255) / 256);
    if (grid > 296) grid = 296;
    tp_push_logits_kernel<<<grid, 256, 0, stream>>>(c, local, slot0, batch, rows, row0, vocab);
  }
  tp_barrier_kernel<<<1, 32, 0, stream>>>(c);
  return launch_status();
}
int bonsai_tp_allgather_logits(void* comm, const float* local, int batch, int rows, int row0, int vocab, cudaStream_t stream) {
  return bonsai_tp_allgather_logits_at(comm, local, 0, batch, rows, row0, vocab, stream);
}
void* bonsai_tp_logits_ptr(void* comm) {
  bonsai::TpComm& c = *static_cast<bonsai::TpComm*>(comm);
  return c.peer[c.rank] + c.lay.off_logits;
}
void* bonsai_tp_big_ptr(void* comm) {
  bonsai::TpComm& c = *static_cast<bonsai::TpComm*>(comm);
  return c.peer[c.rank] + c.lay.off_big;
}

// h[n] += all-reduce(big[n]) where every rank has written its partial sums into its own big area.
int bonsai_tp_allreduce_big_add(void* comm, float* h, size_t n, cudaStream_t stream) {
  using namespace bonsai;
  TpComm& c = *static_cast<TpComm*>(comm);
  if (n % 4 != 0 || n > c.lay.big_elems) return BONSAI_CUDA_BAD_ARG;
  tp_barrier_kernel<<<1, 32, 0, stream>>>(c);
  tp_reduce_broadcast_kernel<<<296, 256, 0, stream>>>(c, n);
  tp_barrier_kernel<<<1, 32, 0, stream>>>(c);
  tp_add_kernel<<<296, 256, 0, stream>>>(h, reinterpret_cast<const float*>(c.peer[c.rank] + c.lay.off_big), n);
  return launch_status();
}

// h[n] += sum over ranks of the partial sums every rank wrote into half `half` (0 or 1) of its big area
// (address: bonsai_tp_big_half_ptr).  One kernel; consecutive calls must alternate halves.
int bonsai_tp_allreduce_oneshot_add(void* comm, float* h, size_t n, int half, cudaStream_t stream) {
  using namespace bonsai;
  TpComm& c = *static_cast<TpComm*>(comm);
  const size_t half_elems = (c.lay.big_elems / 2) & ~(size_t)3;
  if (n % 4 != 0 || n > half_elems || half < 0 || half > 1) return BONSAI_CUDA_BAD_ARG;
  int grid = (int)((n / 4 + 255) / 256);
  if (grid > 148) grid = 148;
  if (grid < 1) grid = 1;
  tp_allreduce_oneshot_add_kernel<<<grid, 256, 0, stream>>>(c, h, n / 4, (size_t)half * half_elems / 4);
  return launch_status();
}
// Multicast mapping of the symmetric buffer (0 = none): switches the stores of the fused epilogues and of the logits
// gather to multimem.st and the sums of the all-reduce kernels to multimem.ld_reduce.
void bonsai_tp_set_multicast(void* comm, uint64_t mc_ptr) {
  static_cast<bonsai::TpComm*>(comm)->mc = reinterpret_cast<uint8_t*>(mc_ptr);
}
int bonsai_tp_has_multicast(void* comm) { return static_cast<bonsai::TpComm*>(comm)->mc != nullptr ? 1 : 0; }
void* bonsai_tp_big_half_ptr(void* comm, int half) {
  bonsai::TpComm& c = *static_cast<bonsai::TpComm*>(comm);
  const size_t half_elems = (c.lay.big_elems / 2) & ~(size_t)3;
  return c.peer[c.rank] + c.lay.off_big + (size_t)half * half_elems * sizeof(float);
}

}  // extern "C"
