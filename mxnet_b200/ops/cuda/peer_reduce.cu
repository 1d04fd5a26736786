// All-reduce of a small fp32 vector over peer memory (NVLink), for sm_100a: the statistics of SyncBatchNorm.
//
// Reference behaviour: src/operator/contrib/sync_batch_norm-inl.h keeps a process-wide shared buffer and a barrier between
// the GPU worker threads of one process.  Here every rank is a process; each owns a slab (cudaMalloc, shared by CUDA IPC):
//
//   uint32 flags[kMaxRanks]              written by peers (index = sender rank): the step each sender has published
//   uint32 status                        set to 1 when a wait ran out (the host reads and clears it)
//   float  data[2][kMaxRanks][cap]       receive area, double-buffered by the parity of the step
//
// One CTA per call: store the local vector into slot [step & 1][rank] of EVERY rank's slab (plain peer stores), make the
// stores visible system-wide, publish the step to every rank's flag, wait (bounded by the global timer) until every rank
// has published this step, then add the slots in rank order, so all ranks compute bit-identical sums.  Two buffers are
// enough: a rank can start step s+2 (which reuses the buffer of step s) only after every rank has published step s+1,
// and a rank publishes s+1 only after its step-s kernel has finished reading.
#include "common.cuh"

namespace mxb {

constexpr int kPeerMaxRanks = 8;

struct PeerReduceParams {
  void* slab[kPeerMaxRanks];     // every rank's slab (own entry = local pointer)
  int rank, nranks;
  int cap;                       // floats per slot
  int n;                         // floats to reduce (n <= cap)
  uint32_t step;                 // increases by one per call, starting at 1
  unsigned long long timeout_ns;
};

constexpr size_t kPeerHeaderBytes = 256;

__device__ __forceinline__ uint32_t* peer_flags(void* slab) { return reinterpret_cast<uint32_t*>(slab); }
__device__ __forceinline__ uint32_t* peer_status(void* slab) { return reinterpret_cast<uint32_t*>(slab) + kPeerMaxRanks; }
__device__ __forceinline__ float* peer_slot(void* slab, int cap, int parity, int sender) {
  return reinterpret_cast<float*>(reinterpret_cast<char*>(slab) + kPeerHeaderBytes) + ((size_t)parity * kPeerMaxRanks + sender) * cap;
}

__global__ void __launch_bounds__(256) peer_allreduce_kernel(const __grid_constant__ PeerReduceParams p, const float* __restrict__ in,
                                                             float* __restrict__ out) {
  const int parity = (int)(p.step & 1u);
  for (int r = 0; r < p.nranks; ++r) {
    float* dst = peer_slot(p.slab[r], p.cap, parity, p.rank);
    for (int i = threadIdx.x; i < p.n; i += blockDim.x) dst[i] = in[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.nranks)
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flags(p.slab[threadIdx.x]) + p.rank), "r"(p.step) : "memory");
  // bounded wait for every rank's flag of this step
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < p.nranks) {
    const uint32_t* flag = peer_flags(p.slab[p.rank]) + threadIdx.x;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    unsigned spins = 0;
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if ((int32_t)(v - p.step) >= 0) break;
      if ((++spins & 63u) == 0) {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > p.timeout_ns) { ok = 0; break; }
        __nanosleep(200);
      }
    }
  }
  __syncthreads();
  if (!ok && threadIdx.x == 0) *peer_status(p.slab[p.rank]) = 1u;
  for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < p.nranks; ++r) acc += __ldcg(peer_slot(p.slab[p.rank], p.cap, parity, r) + i);
    out[i] = acc;
  }
}

}  // namespace mxb

using namespace mxb;

// Bytes of one rank's slab for vectors of up to `cap` floats.
MXB_EXPORT uint64_t mxb_peer_slab_bytes(int cap) {
  return kPeerHeaderBytes + (uint64_t)2 * kPeerMaxRanks * (uint64_t)cap * sizeof(float);
}
MXB_EXPORT int mxb_peer_max_ranks() { return kPeerMaxRanks; }
MXB_EXPORT int mxb_peer_status_offset() { return kPeerMaxRanks * (int)sizeof(uint32_t); }

// slabs: nranks device pointers (peers opened through IPC).  in / out: n floats on this rank's device.
MXB_EXPORT int mxb_peer_allreduce(void* const* slabs, int rank, int nranks, int cap, const float* in, float* out, int n,
                                  uint32_t step, unsigned long long timeout_ns, void* stream) {
  if (nranks < 1 || nranks > kPeerMaxRanks || rank < 0 || rank >= nranks || n < 1 || n > cap || step == 0) return -2;
  PeerReduceParams p;
  for (int r = 0; r < kPeerMaxRanks; ++r) p.slab[r] = r < nranks ? slabs[r] : nullptr;
  p.rank = rank; p.nranks = nranks; p.cap = cap; p.n = n; p.step = step; p.timeout_ns = timeout_ns;
  peer_allreduce_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(p, in, out);
  return (int)cudaGetLastError();
}
