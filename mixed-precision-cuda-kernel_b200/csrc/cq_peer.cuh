// Device side of the exchange over peer memory (protocol and region layout: cq_peer.cu), shared by
// the stand-alone kernel there and by the decode kernel, whose last CTA runs the exchange itself.
#pragma once
#include "cq_common.cuh"

namespace cq_peer {

constexpr int MAX_RANKS = 8;
// region header: this rank's call counter at byte 0, the capacity the region was created with at byte 8, the
// decode kernel's CTA arrival counter at byte 64
constexpr size_t EPOCH_OFF = 0, CAPACITY_OFF = 8, DONE_OFF = 64, LANDING_OFF = 256;

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

// One call of the exchange by the THREADS threads of a CTA (all of them must call it; s_fail is a
// shared-memory word).  The slice x may have been written by other CTAs of the same grid (the caller has
// fenced): it is read past L1.
template <int THREADS>
__device__ __forceinline__ void exchange(const PeerGatherParams& p, int* s_fail) {
  const uint32_t tid = threadIdx.x;
  if (tid == 0) *s_fail = 0;
  uint8_t* own = nullptr;
#pragma unroll
  for (int r = 0; r < MAX_RANKS; ++r)
    if (r == p.rank) own = p.region[r];
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(own + EPOCH_OFF) + 1u;
  const size_t area = LANDING_OFF + (size_t)(e & 1u) * p.capacity;
  // a call whose capacity is not the one the region was created with would address the landing areas wrongly:
  // nothing is sent, the call ends like one whose peers never delivered
  const bool geometry_ok = *reinterpret_cast<volatile unsigned long long*>(own + CAPACITY_OFF) == p.capacity;

  // 1. deliver the own slice to every rank (this one included): 8 payload bytes -> 16 bytes {d0, e, d1, e}
  for (uint32_t i = tid; geometry_ok && i < p.slice8; i += THREADS) {
    const uint2 d = __ldcg(p.x + i);
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
  bool failed = !geometry_ok;
  for (uint32_t idx = tid; idx < total && !failed; idx += THREADS) {
    for (;;) {
      const uint4 w = ld_landing(land + idx);
      if (w.y == e && w.w == e) break;
      if (now_ns() - t0 > p.wait_ns) {
        failed = true;
        break;
      }
    }
  }
  if (failed) *s_fail = 1;
  __syncthreads();
  if (*s_fail) {
    // a peer never delivered: report, keep the call counter in step, and fill the whole output with
    // NaN so that nothing downstream can take stale memory for a result
    for (uint32_t idx = tid; idx < total; idx += THREADS) p.out[idx] = make_uint2(0x7e007e00u, 0x7e007e00u);
    if (tid == 0) {
      if (p.status) atomicOr(p.status, (uint32_t)CQ_ERR_DEVICE_TIMEOUT);
      *reinterpret_cast<volatile uint32_t*>(own + EPOCH_OFF) = e;
    }
    return;
  }

  // 3. landing[rank r][row][unit] -> out[row][r][unit]   (every word is known to be complete now)
  for (uint32_t idx = tid; idx < total; idx += THREADS) {
    const uint32_t r = idx / p.slice8, i = idx - r * p.slice8;
    const uint32_t row = i / p.row8, u = i - row * p.row8;
    const uint4 w = ld_landing(land + idx);
    p.out[((size_t)row * p.world + r) * p.row8 + u] = make_uint2(w.x, w.z);
  }
  if (tid == 0) *reinterpret_cast<volatile uint32_t*>(own + EPOCH_OFF) = e;
}

// Fills the geometry of a call; returns a status code.
inline int fill_params(PeerGatherParams* p, void* const* regions, int world, int rank, size_t capacity, const void* x_f16,
                       void* out_f16, int rows, int cols_local, int timeout_ms, uint32_t* status_word) {
  if (!regions || !x_f16 || !out_f16 || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || rows < 1 ||
      cols_local < 8 || timeout_ms < 1 || timeout_ms > 60000)
    return CQ_ERR_BAD_ARG;
  if (cols_local & 7) return CQ_ERR_BAD_SHAPE;                       // 8-byte units never straddle a row
  if (((uintptr_t)x_f16 | (uintptr_t)out_f16) & 7) return CQ_ERR_BAD_ARG;
  const unsigned long long slice = (unsigned long long)rows * cols_local * 2ull;
  // on the wire every 8 payload bytes take 16
  if (2 * slice * world > capacity || slice * world > 0x3fffffffull) return CQ_ERR_TOO_LARGE;
  *p = PeerGatherParams{};
  for (int r = 0; r < world; ++r) {
    if (!regions[r] || ((uintptr_t)regions[r] & 15)) return CQ_ERR_BAD_ARG;
    p->region[r] = static_cast<uint8_t*>(regions[r]);
  }
  p->x = static_cast<const uint2*>(x_f16);
  p->out = static_cast<uint2*>(out_f16);
  p->status = status_word;
  p->capacity = capacity;
  p->wait_ns = (unsigned long long)timeout_ms * 1000000ull;
  p->slice8 = (uint32_t)(slice / 8);
  p->row8 = (uint32_t)(cols_local / 4);
  p->world = world;
  p->rank = rank;
  return CQ_OK;
}

}  // namespace cq_peer
