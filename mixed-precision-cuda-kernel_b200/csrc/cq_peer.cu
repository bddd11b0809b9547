// All-gather of the column-parallel output slices over peer memory (NVLink / NVSwitch), as one small
// kernel per rank instead of a library collective.  The reference has no multi-GPU path; this is
// the exchange step of the column-parallel quantized linear (every rank holds N / P output rows of
// a layer and needs the whole output vector for the next layer).
//
// Every rank owns one "region" of device memory that its peers map through CUDA IPC:
//
//   byte 0     epoch uint32                      this rank's own call counter (peers never touch it)
//   byte 8     capacity uint64                   bytes of one landing area, checked by every call against its argument
//   byte 64    done uint32                       arrivals of the CTAs of a decode kernel that ends with the exchange
//   byte 256   landing[0]  (capacity bytes)      slices of even epochs, [rank][8-byte words]
//   ...        landing[1]  (capacity bytes)      slices of odd epochs
//
// The exchange is latency-bound (a few KB per rank), so data and arrival flag travel together:
// every 8-byte word on the wire is {4 bytes of payload, the call's epoch number}.  A call with
// epoch e (every rank makes the same sequence of calls) stores its slice in that form into
// landing[e & 1][rank] of every rank with plain peer stores, then polls the words of its own landing
// area until each carries e (bounded by the caller's time limit) and writes the payloads to the
// caller's (rows, P * cols_local) output.  No fence, no separate flag, one NVLink crossing.  An 8-byte
// aligned store arrives whole, so a word whose second half reads e has its payload; stale words hold
// older epochs (or zero, from creation) and never match.
// The two landing areas make re-use safe without a second handshake: a peer can only write epoch
// e + 2 into the area of epoch e after its call e + 1 has finished, which needs this rank's words of
// e + 1, and this rank sends those in a kernel that runs after its read-out of epoch e (stream order).
//
// The wait is on kernels of OTHER GPUs, one rank per GPU; ranks must not share a device.  No
// multicast, no TMA: plain loads and stores on mapped peer memory.
#include "cq_common.cuh"
#include "cq_peer.cuh"

namespace {

using namespace cq_peer;
constexpr int GATHER_THREADS = 1024;

__global__ void __launch_bounds__(GATHER_THREADS) peer_allgather_kernel(const PeerGatherParams p) {
  __shared__ int s_fail;
  // the slice comes from the kernel launched before this one
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  exchange<GATHER_THREADS>(p, &s_fail);
}

}  // namespace

extern "C" size_t cq_peer_region_bytes(size_t capacity) { return LANDING_OFF + 2 * capacity; }

extern "C" int cq_peer_region_create(size_t capacity, void** region) {
  if (!region || capacity < 16 || (capacity & 15)) return CQ_ERR_BAD_ARG;
  void* p = nullptr;
  CQ_CUDA_TRY(cudaMalloc(&p, cq_peer_region_bytes(capacity)));
  cudaError_t e = cudaMemset(p, 0, cq_peer_region_bytes(capacity));
  const unsigned long long cap = capacity;
  if (e == cudaSuccess) e = cudaMemcpy((uint8_t*)p + CAPACITY_OFF, &cap, sizeof(cap), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(p);
    CQ_CUDA_TRY(e);
  }
  *region = p;
  return CQ_OK;
}

extern "C" int cq_peer_region_destroy(void* region) {
  if (!region) return CQ_ERR_BAD_ARG;
  CQ_CUDA_TRY(cudaFree(region));
  return CQ_OK;
}

extern "C" int cq_peer_region_export(const void* region, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (!region || !handle) return CQ_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  CQ_CUDA_TRY(cudaIpcGetMemHandle(&h, const_cast<void*>(region)));
  memcpy(handle, &h, sizeof(h));
  return CQ_OK;
}

extern "C" int cq_peer_region_open(const unsigned char handle[64], void** region) {
  if (!region || !handle) return CQ_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  CQ_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *region = p;
  return CQ_OK;
}

extern "C" int cq_peer_region_close(void* region) {
  if (!region) return CQ_ERR_BAD_ARG;
  CQ_CUDA_TRY(cudaIpcCloseMemHandle(region));
  return CQ_OK;
}

extern "C" int cq_peer_allgather(void* const* regions, int world, int rank, size_t capacity, const void* x_f16,
                                 void* out_f16, int rows, int cols_local, int timeout_ms,
                                 uint32_t* status_word, cq_stream_t stream) {
  PeerGatherParams p;
  const int rc = fill_params(&p, regions, world, rank, capacity, x_f16, out_f16, rows, cols_local, timeout_ms, status_word);
  if (rc != CQ_OK) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(GATHER_THREADS);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, peer_allgather_kernel, p));
  return CQ_OK;
}
