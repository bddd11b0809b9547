// All-gather of the column-parallel output slices over peer memory (NVLink / NVSwitch), as one small
// kernel per rank instead of a library collective.  The reference has no multi-GPU path; this is
// the exchange step of the column-parallel quantized linear (every rank holds N / P output rows of
// a layer and needs the whole output vector for the next layer).
//
// Every rank owns one "region" of device memory that its peers map through CUDA IPC:
//
//   byte 0     epoch uint32                      this rank's own call counter (peers never touch it)
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

namespace {

constexpr int MAX_RANKS = 8;
constexpr size_t EPOCH_OFF = 0, LANDING_OFF = 256;
constexpr int GATHER_THREADS = 1024;

struct PeerGatherParams {
  uint8_t* region[MAX_RANKS];     // region[rank] is this rank's own
  const uint2* x;                 // (rows, cols_local) fp16, contiguous, read 8 bytes at a time
  uint2* out;                     // (rows, world * cols_local) fp16, contiguous
  uint32_t* status;               // may be null
  unsigned long long capacity;    // bytes of one landing area
  unsigned long long wait_ns;     // limit of the wait for the peers
  uint32_t slice8;                // 8-byte payload units of one rank's slice
  uint32_t row8;                  // 8-byte payload units of one row of a slice
  int world, rank;
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint4 ld_landing(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(GATHER_THREADS) peer_allgather_kernel(const PeerGatherParams p) {
  __shared__ int s_fail;
  // the slice comes from the kernel launched before this one
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t tid = threadIdx.x;
  if (tid == 0) s_fail = 0;
  uint8_t* own = nullptr;
#pragma unroll
  for (int r = 0; r < MAX_RANKS; ++r)
    if (r == p.rank) own = p.region[r];
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(own + EPOCH_OFF) + 1u;
  const size_t area = LANDING_OFF + (size_t)(e & 1u) * p.capacity;

  // 1. deliver the own slice to every rank (this one included): 8 payload bytes -> 16 bytes {d0, e, d1, e}
  for (uint32_t i = tid; i < p.slice8; i += GATHER_THREADS) {
    const uint2 d = p.x[i];
    const uint4 w = make_uint4(d.x, e, d.y, e);
    const size_t at = area + ((size_t)p.rank * p.slice8 + i) * 16;
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r)
      if (r < p.world) *reinterpret_cast<uint4*>(p.region[r] + at) = w;
  }
  __syncthreads();                       // (s_fail is initialised)

  // 2. wait until every word of the own landing area carries this epoch (bounded)
  const uint4* land = reinterpret_cast<const uint4*>(own + area);
  const uint32_t total = p.slice8 * (uint32_t)p.world;
  const unsigned long long t0 = now_ns();
  bool failed = false;
  for (uint32_t idx = tid; idx < total && !failed; idx += GATHER_THREADS) {
    for (;;) {
      const uint4 w = ld_landing(land + idx);
      if (w.y == e && w.w == e) break;
      if (now_ns() - t0 > p.wait_ns) {
        failed = true;
        break;
      }
    }
  }
  if (failed) s_fail = 1;
  __syncthreads();
  if (s_fail) {
    // a peer never delivered: report, keep the call counter in step, and fill the whole output with
    // NaN so that nothing downstream can take stale memory for a result
    for (uint32_t idx = tid; idx < total; idx += GATHER_THREADS) p.out[idx] = make_uint2(0x7e007e00u, 0x7e007e00u);
    if (tid == 0) {
      if (p.status) atomicOr(p.status, (uint32_t)CQ_ERR_DEVICE_TIMEOUT);
      *reinterpret_cast<volatile uint32_t*>(own + EPOCH_OFF) = e;
    }
    return;
  }

  // 3. landing[rank r][row][unit] -> out[row][r][unit]   (every word is known to be complete now)
  for (uint32_t idx = tid; idx < total; idx += GATHER_THREADS) {
    const uint32_t r = idx / p.slice8, i = idx - r * p.slice8;
    const uint32_t row = i / p.row8, u = i - row * p.row8;
    const uint4 w = ld_landing(land + idx);
    p.out[((size_t)row * p.world + r) * p.row8 + u] = make_uint2(w.x, w.z);
  }
  if (tid == 0) *reinterpret_cast<volatile uint32_t*>(own + EPOCH_OFF) = e;
}

}  // namespace

extern "C" size_t cq_peer_region_bytes(size_t capacity) { return LANDING_OFF + 2 * capacity; }

extern "C" int cq_peer_region_create(size_t capacity, void** region) {
  if (!region || capacity < 16 || (capacity & 15)) return CQ_ERR_BAD_ARG;
  void* p = nullptr;
  CQ_CUDA_TRY(cudaMalloc(&p, cq_peer_region_bytes(capacity)));
  cudaError_t e = cudaMemset(p, 0, cq_peer_region_bytes(capacity));
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
  if (!regions || !x_f16 || !out_f16 || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || rows < 1 ||
      cols_local < 8 || timeout_ms < 1 || timeout_ms > 60000)
    return CQ_ERR_BAD_ARG;
  if (cols_local & 7) return CQ_ERR_BAD_SHAPE;                       // 8-byte units never straddle a row
  if (((uintptr_t)x_f16 | (uintptr_t)out_f16) & 7) return CQ_ERR_BAD_ARG;
  const unsigned long long slice = (unsigned long long)rows * cols_local * 2ull;
  // on the wire every 8 payload bytes take 16
  if (2 * slice * world > capacity || slice * world > 0x3fffffffull) return CQ_ERR_TOO_LARGE;
  PeerGatherParams p = {};
  for (int r = 0; r < world; ++r) {
    if (!regions[r] || ((uintptr_t)regions[r] & 15)) return CQ_ERR_BAD_ARG;
    p.region[r] = static_cast<uint8_t*>(regions[r]);
  }
  p.x = static_cast<const uint2*>(x_f16);
  p.out = static_cast<uint2*>(out_f16);
  p.status = status_word;
  p.capacity = capacity;
  p.wait_ns = (unsigned long long)timeout_ms * 1000000ull;
  p.slice8 = (uint32_t)(slice / 8);
  p.row8 = (uint32_t)(cols_local / 4);
  p.world = world;
  p.rank = rank;
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
