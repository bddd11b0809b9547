// Row-layout decode matvec: y (1, N) fp16 = [y +] x (1, K) fp16 . W^T for ONE activation row.
//
// Replaces the reference's batch-1 use of VecQuant4MatMulKernelCherryQBatchedHalf and
// VecQuant3MatMulKernelCherryQBatched(G64)Half (csrc/quant_cuda_kernel.cu:718-835, 558-672,
// 316-438 of the reference project): one thread per output column there, byte loads at stride N,
// fp16 atomics.  Here:
//
//   * layout: every output row is one contiguous record (cq_rlayer, include/cherryq.h).  A CTA
//     owns a contiguous range of rows, i.e. one contiguous byte range of the layer, a warp owns
//     whole rows, lane l owns the 128 compact columns of group l of its K slice;
//   * the CTA's byte range is requested with a handful of bulk async copies (cp.async.bulk +
//     mbarrier transaction counts) into shared memory the moment the CTA starts, BEFORE it waits
//     for the previous kernel in the stream (programmatic dependent launch): weights are
//     constants, only x is not.  HBM streams while the activations are staged; the rows are then
//     read from shared memory with conflict-free 16-byte loads.  Rows beyond the shared-memory
//     capacity (large layers) are read from global memory with a register pipeline D rows deep;
//   * the activations of a lane never change from row to row: they sit in registers for the whole
//     kernel as two signed-byte planes (q = 128 hi + lo, |q| <= 16256, one step size per group),
//     so a row costs two masks and four integer dot products (dp4a, u8 x s8) per 8 weights:
//         sum_k (u_k - off) x_k = sx (sum u q - off sum q),  sum u q exact in 32-bit integers;
//   * no cross-CTA traffic, no atomics, no scratch: a row's partial sums meet in one warp
//     (shuffles) or, for K > 4096 (several slices), in the CTA's shared memory, in a fixed order.
#include "cq_common.cuh"

namespace {

constexpr int RV_NBAR = 32;                 // mbarriers (groups of row iterations) per CTA
constexpr uint32_t RV_WAIT_LIMIT = 1u << 22;

struct RowvecParams {
  const uint8_t* rows;      // records: [codes row_bytes][scales srow_bytes][cherry 2 C]
  const uint16_t* perm;
  const uint16_t* cidx;
  const __half* x;
  __half* y;
  uint32_t* status;         // may be null
  int K, N, C, NG, nsl, gps, cps, accumulate;
  int row_bytes, srow_bytes, rec_bytes;
  int rows_q, rows_r;       // CTA b owns rows_q (+1 if b < rows_r) consecutive rows
  int smem_rows;            // rows of a CTA that fit its shared-memory row area
  int pre_pct;              // share (percent) of the shared-memory rows requested before the dependency wait
  int l2_prefetch;          // the rest is asked into L2 at once (1) or not (0)
  int off_planes, off_sx, off_part, off_bar, off_rows;    // shared-memory sections (bytes)
#ifdef CQ_ROWVEC_TRACE
  int trace_launch;
#endif
};

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t rv_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void rv_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void rv_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool rv_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait (polls and about one second of the nanosecond timer); on failure the CTA-wide
// abort flag makes every later wait give up at once, bit 0 of the status word is set and the
// kernel runs on to its normal exit.
__device__ __noinline__ bool rv_mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t* status) {
  const uint32_t limit = *abort_flag ? 1u : RV_WAIT_LIMIT;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t it = 0; it < limit; ++it) {
    if (rv_mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 63u) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > 1000000000ull) break;
    }
  }
  *abort_flag = 1;
  if (status) atomicOr(status, 1u);
  return false;
}
__device__ __forceinline__ bool rv_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t* status) {
  if (rv_mbar_try_wait(bar, parity)) return true;
  return rv_mbar_wait_slow(bar, parity, abort_flag, status);
}
__device__ __forceinline__ void rv_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream4(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream2(const void* p) {
  uint16_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ float h2f_bits(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// 16 x sum over one half group (64 columns) of u_k q_k, for both halves of a lane's 128 columns.
//   4-bit word w (columns 8w .. 8w+7): low nibbles of its bytes = columns 8w..8w+3, high nibbles =
//   columns 8w+4..8w+7; the high nibbles are used where they are (16 u), hence the factor 16.
//   3-bit words A, B, C of a 32-column set: bits 0-2 / 4-6 of byte b = columns 4f + b of fields
//   f = 0..5, bit 3 / bit 7 of the three words = bit planes of fields 6 / 7.
template <int BITS>
__device__ __forceinline__ void dot_halves(const uint32_t (&w)[4 * BITS], const int (&xh)[32], const int (&xl)[32],
                                           int (&t)[2]) {
  int a1h[2] = {0, 0}, a1l[2] = {0, 0}, a16h[2] = {0, 0}, a16l[2] = {0, 0};
#ifdef CQ_ROWVEC_NOCOMPUTE   // tuning builds: loads only
  {
    uint32_t v = 0;
#pragma unroll
    for (int i = 0; i < 4 * BITS; ++i) v ^= w[i];
    t[0] = (int)v + xh[0]; t[1] = xl[0];
    return;
  }
#endif
  if (BITS == 4) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int h = i >> 3;
      const uint32_t lo = w[i] & 0x0F0F0F0Fu, hi = w[i] & 0xF0F0F0F0u;
      a1h[h] = dp4a_us(lo, xh[2 * i], a1h[h]);
      a1l[h] = dp4a_us(lo, xl[2 * i], a1l[h]);
      a16h[h] = dp4a_us(hi, xh[2 * i + 1], a16h[h]);
      a16l[h] = dp4a_us(hi, xl[2 * i + 1], a16l[h]);
    }
  } else {
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int h = s >> 1, xb = 8 * s;
      const uint32_t A = w[3 * s], B = w[3 * s + 1], Cw = w[3 * s + 2];
      const uint32_t f0 = A & 0x07070707u, f1 = A & 0x70707070u;
      const uint32_t f2 = B & 0x07070707u, f3 = B & 0x70707070u;
      const uint32_t f4 = Cw & 0x07070707u, f5 = Cw & 0x70707070u;
      const uint32_t f6 = ((A >> 3) & 0x01010101u) | ((B >> 2) & 0x02020202u) | ((Cw >> 1) & 0x04040404u);
      const uint32_t f7 = ((A >> 7) & 0x01010101u) | ((B >> 6) & 0x02020202u) | ((Cw >> 5) & 0x04040404u);
      a1h[h] = dp4a_us(f0, xh[xb + 0], a1h[h]);   a1l[h] = dp4a_us(f0, xl[xb + 0], a1l[h]);
      a16h[h] = dp4a_us(f1, xh[xb + 1], a16h[h]); a16l[h] = dp4a_us(f1, xl[xb + 1], a16l[h]);
      a1h[h] = dp4a_us(f2, xh[xb + 2], a1h[h]);   a1l[h] = dp4a_us(f2, xl[xb + 2], a1l[h]);
      a16h[h] = dp4a_us(f3, xh[xb + 3], a16h[h]); a16l[h] = dp4a_us(f3, xl[xb + 3], a16l[h]);
      a1h[h] = dp4a_us(f4, xh[xb + 4], a1h[h]);   a1l[h] = dp4a_us(f4, xl[xb + 4], a1l[h]);
      a16h[h] = dp4a_us(f5, xh[xb + 5], a16h[h]); a16l[h] = dp4a_us(f5, xl[xb + 5], a16l[h]);
      a1h[h] = dp4a_us(f6, xh[xb + 6], a1h[h]);   a1l[h] = dp4a_us(f6, xl[xb + 6], a1l[h]);
      a1h[h] = dp4a_us(f7, xh[xb + 7], a1h[h]);   a1l[h] = dp4a_us(f7, xl[xb + 7], a1l[h]);
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) t[h] = ((a1h[h] * 128 + a1l[h]) << 4) + (a16h[h] * 128 + a16l[h]);
}

#ifdef CQ_ROWVEC_TRACE   // tuning builds: %globaltimer stamps per CTA, buffer [16 launches][1024 CTAs][16]
__device__ unsigned long long* cq_rv_trace = nullptr;
__device__ __forceinline__ void rv_stamp(int launch, int slot) {
  if (cq_rv_trace && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    cq_rv_trace[((size_t)(launch & 15) * 1024 + blockIdx.x) * 16 + slot] = t;
  }
}
#define RV_STAMP(s) rv_stamp(p.trace_launch, s)
#else
#define RV_STAMP(s)
#endif

// Quantises octet o of the compact activations (columns `cols` of the fp16 row in shared memory)
// and stores its bytes of the two planes; the first thread of a group also stores the group's
// step and offset terms.  All 32 lanes of a warp call it.
template <int SETS>
__device__ __forceinline__ void stage_octet(const __half* raw, const uint4 cols, int o, int n_oct, int NG, float OFF,
                                            unsigned char* planes, float* gsx, float* gcq) {
  const uint32_t pw[4] = {cols.x, cols.y, cols.z, cols.w};
  float v[8];
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t col = (pw[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
    v[i] = __half2float(raw[col]);                 // padding columns point at the zero slot raw[K]
    m = fmaxf(m, fabsf(v[i]));
  }
#pragma unroll
  for (int s = 1; s < 16; s <<= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, s));
  const float step = m * (1.0f / 16256.0f);
  const float inv = m > 0.f ? 16256.0f / m : 0.f;
  uint32_t hi[8], lo[8];
  int sq = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int q = __float2int_rn(v[i] * inv);
    const int t = q + 64;
    hi[i] = (uint32_t)(t >> 7);                    // floor((q + 64) / 128) in [-127, 127]
    lo[i] = (uint32_t)((t & 127) - 64);            // q - 128 hi in [-64, 63]
    sq += q;
  }
  uint32_t hw[2], lw[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {                    // low bytes of four values -> one word
    hw[k] = __byte_perm(__byte_perm(hi[4 * k], hi[4 * k + 1], 0x0040), __byte_perm(hi[4 * k + 2], hi[4 * k + 3], 0x0040), 0x5410);
    lw[k] = __byte_perm(__byte_perm(lo[4 * k], lo[4 * k + 1], 0x0040), __byte_perm(lo[4 * k + 2], lo[4 * k + 3], 0x0040), 0x5410);
  }
  // sums of q over the two 64-column halves of the group
  sq += __shfl_xor_sync(0xFFFFFFFFu, sq, 1);
  sq += __shfl_xor_sync(0xFFFFFFFFu, sq, 2);
  sq += __shfl_xor_sync(0xFFFFFFFFu, sq, 4);
  const int sq_other = __shfl_xor_sync(0xFFFFFFFFu, sq, 8);
  if (o < n_oct) {
    const int gg = o >> 4, oo = o & 15;
    unsigned char* dst = planes + ((size_t)(oo >> 1) * NG + gg) * 16 + (oo & 1) * 8;
    *reinterpret_cast<uint2*>(dst) = make_uint2(hw[0], hw[1]);
    *reinterpret_cast<uint2*>(dst + (size_t)8 * NG * 16) = make_uint2(lw[0], lw[1]);
    if (oo == 0) {
      gsx[gg] = step * (1.0f / 16.0f);
      if (SETS == 2) {
        gcq[2 * gg] = -OFF * step * (float)sq;
        gcq[2 * gg + 1] = -OFF * step * (float)sq_other;
      } else {
        gcq[gg] = -OFF * step * (float)(sq + sq_other);
      }
    }
  }
}

// One row of one lane: the integer dot products, the group's scale(s), the cherry product.
template <int BITS, int SETS>
__device__ __forceinline__ float row_value(const uint32_t (&w)[4 * BITS], uint32_t scw, uint32_t chw, const int (&xh)[32],
                                           const int (&xl)[32], float sx16, float cq0, float cq1, float xc, bool lane_on) {
  int t[2];
  dot_halves<BITS>(w, xh, xl, t);
  float acc;
  if (SETS == 2) {
    acc = h2f_bits(scw & 0xFFFFu) * fmaf((float)t[0], sx16, cq0) + h2f_bits(scw >> 16) * fmaf((float)t[1], sx16, cq1);
  } else {
    acc = h2f_bits(scw & 0xFFFFu) * fmaf((float)(t[0] + t[1]), sx16, cq0);
  }
  acc = lane_on ? acc : 0.f;
  return fmaf(h2f_bits(chw & 0xFFFFu), xc, acc);
}

// Sums R per-lane values over the 32 lanes; afterwards lane (32 / R) * r holds the total of value r.
template <int R>
__device__ __forceinline__ float reduce_rows(const float (&acc)[R], int lane) {
  if (R == 4) {
    const bool b4 = lane & 16, b3 = lane & 8;
    float a = (b4 ? acc[2] : acc[0]) + __shfl_xor_sync(0xFFFFFFFFu, b4 ? acc[0] : acc[2], 16);
    float b = (b4 ? acc[3] : acc[1]) + __shfl_xor_sync(0xFFFFFFFFu, b4 ? acc[1] : acc[3], 16);
    float c = (b3 ? b : a) + __shfl_xor_sync(0xFFFFFFFFu, b3 ? a : b, 8);
    c += __shfl_xor_sync(0xFFFFFFFFu, c, 4);
    c += __shfl_xor_sync(0xFFFFFFFFu, c, 2);
    c += __shfl_xor_sync(0xFFFFFFFFu, c, 1);
    return c;
  } else if (R == 2) {
    const bool b4 = lane & 16;
    float c = (b4 ? acc[1] : acc[0]) + __shfl_xor_sync(0xFFFFFFFFu, b4 ? acc[0] : acc[1], 16);
#pragma unroll
    for (int s = 8; s >= 1; s >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, s);
    return c;
  } else {
    float c = acc[0];
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, s);
    return c;
  }
}

// Requests the CTA's records of barriers [b0, b1) from global memory, in the order the warps
// consume them; one thread calls it.
__device__ __noinline__ void issue_rows(const RowvecParams& p, unsigned char* srows, uint32_t bar0, int r0, int n_smem,
                                        int rows_per_bar, int b0, int b1) {
  const uint8_t* src = p.rows + (size_t)r0 * p.rec_bytes;
  const uint32_t dst = rv_smem_u32(srows);
  for (int b = b0; b < b1; ++b) {
    const int ra = b * rows_per_bar, rb = min(n_smem, ra + rows_per_bar);
    const uint32_t bytes = (uint32_t)(rb - ra) * p.rec_bytes;
    rv_mbar_expect_tx(bar0 + 8 * b, bytes);
    for (uint32_t off = 0; off < bytes; off += 32768) {
      const uint32_t sz = bytes - off < 32768 ? bytes - off : 32768;
      rv_bulk_g2s(dst + (uint32_t)ra * p.rec_bytes + off, src + (size_t)ra * p.rec_bytes + off, sz, bar0 + 8 * b);
    }
  }
}

// BITS 3 | 4; SETS scale sets per 128 columns (2 for 64-wide groups); W warps per CTA;
// D rows of a lane in flight on the global-memory path (0: the kernel has no such path and every
// row of the CTA must fit shared memory); R rows of a warp are worked on together.
template <int BITS, int SETS, int W, int D, int R>
__global__ void __launch_bounds__(W * 32, 1) cq_rowvec_kernel(const RowvecParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_abort;
  constexpr int J = BITS;              // 16-byte chunks per lane and row
  constexpr int NW = 4 * BITS;         // 32-bit words per lane and row
  constexpr int NTHR = W * 32;
  constexpr int DG = D > 0 ? D : 1;
  constexpr float OFF = BITS == 4 ? 7.5f : 3.5f;
  constexpr int PV = 4;                // octets of activations a thread stages with preloaded column lists
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  RV_STAMP(0);

  __half* raw = reinterpret_cast<__half*>(smem);
  unsigned char* planes = smem + p.off_planes;
  float* gsx = reinterpret_cast<float*>(smem + p.off_sx);   // [NG]      step / 16 of the group's activations
  float* gcq = gsx + p.NG;                                   // [NG][SETS] -off * step * sum q
  float* part = reinterpret_cast<float*>(smem + p.off_part);
  const uint32_t bar0 = rv_smem_u32(smem + p.off_bar);
  unsigned char* srows = smem + p.off_rows;

  const int NG = p.NG, nsl = p.nsl;
  const int r0 = (int)blockIdx.x * p.rows_q + min((int)blockIdx.x, p.rows_r);
  const int r1 = r0 + p.rows_q + ((int)blockIdx.x < p.rows_r ? 1 : 0);
  const int RL = W / nsl;                         // warps that work on different rows at a time
  const int n_smem = min(r1 - r0, p.smem_rows);   // rows of this CTA that go through shared memory
  // rows are handed out in iterations of RL rows; a barrier covers `ipb` iterations
  const int smem_iters = (n_smem + RL - 1) / RL;
  const int ipb = max(1, (smem_iters + RV_NBAR - 1) / RV_NBAR);

  const int rows_per_bar = ipb * RL;
  const int nbar = (n_smem + rows_per_bar - 1) / rows_per_bar;      // barriers in use
  const int nbar_pre = (nbar * p.pre_pct + 99) / 100;               // ... requested before the wait
  if (tid == 0) {
    s_abort = 0;
    for (int b = 0; b < RV_NBAR; ++b) rv_mbar_init(bar0 + 8 * b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    issue_rows(p, srows, bar0, r0, n_smem, rows_per_bar, 0, nbar_pre);
  }
  if (p.l2_prefetch && nbar_pre < nbar) {
    // the records that are copied after the wait: ask for them to be brought into L2 meanwhile
    const uint8_t* lo = p.rows + ((size_t)r0 + (size_t)nbar_pre * rows_per_bar) * p.rec_bytes;
    const uint8_t* hi = p.rows + ((size_t)r0 + n_smem) * p.rec_bytes;
    for (const uint8_t* a = lo + (size_t)tid * 128; a < hi; a += (size_t)NTHR * 128)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
  }

  const int sl = warp % nsl, rl = warp / nsl;     // K slice and row lane of this warp
  const int g0 = sl * p.gps;
  const int gcount = min(p.gps, NG - g0);
  const bool lane_on = lane < gcount;
  const int g = lane_on ? g0 + lane : g0;
  const int c0 = sl * p.cps;
  const bool cher_on = lane < min(p.cps, p.C - c0);
  const int nrows = rl < RL ? max(0, (r1 - r0 - rl + RL - 1) / RL) : 0;          // rows of this warp
  const int nrows_s = rl < RL ? max(0, (n_smem - rl + RL - 1) / RL) : 0;        // ... of which from shared memory

  // byte offsets inside a record
  const int woff = g0 * (16 * BITS) + (lane_on ? lane : 0) * 16;   // idle lanes re-read lane 0's bytes and drop the result
  const int jstride = gcount * 16;
  const int soff = p.row_bytes + g * (2 * SETS);
  const int coff = cher_on ? p.row_bytes + p.srow_bytes + (c0 + lane) * 2 : 0;   // lanes without a cherry read code bytes and ignore them

  // global-memory path: request the first D of its rows now
  const uint8_t* gptr = p.rows + ((size_t)r0 + rl + (size_t)nrows_s * RL) * p.rec_bytes;
  const size_t gstep = (size_t)RL * p.rec_bytes;
  const int nrows_g = nrows - nrows_s;
  uint4 wb[DG][J];
  uint32_t sc[DG], ch[DG];
  if (D > 0) {
#pragma unroll
    for (int d = 0; d < DG; ++d) {
      sc[d] = 0; ch[d] = 0;
#pragma unroll
      for (int j = 0; j < J; ++j) wb[d][j] = make_uint4(0, 0, 0, 0);
      if (d < nrows_g) {
        const uint8_t* rp = gptr + d * gstep;
        if (lane_on) {
#pragma unroll
          for (int j = 0; j < J; ++j) wb[d][j] = ldg_stream16(rp + woff + j * jstride);
          sc[d] = SETS == 2 ? ldg_stream4(rp + soff) : ldg_stream2(rp + soff);
        }
        if (cher_on) ch[d] = ldg_stream2(rp + coff);
      }
    }
  }
  // layer constants of the activation staging: the column lists of this thread's first PV octets
  const int n_oct = NG * 16;
  const uint32_t padpair = (uint32_t)p.K * 0x10001u;
  const uint4 padcols = make_uint4(padpair, padpair, padpair, padpair);
  uint4 pv[PV];
#pragma unroll
  for (int u = 0; u < PV; ++u) {
    const int o = u * NTHR + tid;
    pv[u] = padcols;
    if (o < n_oct) pv[u] = *reinterpret_cast<const uint4*>(p.perm + (size_t)o * 8);
  }
  const int ccol = cher_on ? p.cidx[c0 + lane] : 0;

  RV_STAMP(1);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  RV_STAMP(2);

  // ---- activations: the fp16 row goes to shared memory with coalesced 16-byte loads, then every
  // thread quantises octets of compact columns: one step size per group (16 consecutive threads),
  // two signed-byte planes.
  if ((reinterpret_cast<uintptr_t>(p.x) & 15) == 0) {
    for (int i = tid; i < p.K / 8; i += NTHR)
      reinterpret_cast<uint4*>(raw)[i] = __ldcg(reinterpret_cast<const uint4*>(p.x) + i);
  } else {
    for (int i = tid; i < p.K; i += NTHR) raw[i] = p.x[i];
  }
  if (tid < 8) raw[p.K + tid] = __float2half(0.f);
  if (tid == 0 && nbar_pre < nbar) issue_rows(p, srows, bar0, r0, n_smem, rows_per_bar, nbar_pre, nbar);
  __syncthreads();
  RV_STAMP(6);
  const float xc = cher_on ? __half2float(raw[ccol]) : 0.f;
#pragma unroll 1
  for (int u = 0; u * NTHR < n_oct; ++u) {
    const int o = u * NTHR + tid;
    uint4 pw = u == 0 ? pv[0] : (u == 1 ? pv[1] : (u == 2 ? pv[2] : pv[3]));
    if (u >= PV) {
      pw = padcols;
      if (o < n_oct) pw = *reinterpret_cast<const uint4*>(p.perm + (size_t)o * 8);
    }
    RV_STAMP(8);
#ifndef CQ_ROWVEC_NOSTAGE   // tuning builds can leave the quantisation out to count its instructions
    stage_octet<SETS>(raw, pw, o, n_oct, NG, OFF, planes, gsx, gcq);
#else
    if (o == 0x7fffffff) planes[0] = (unsigned char)pw.x;
#endif
    RV_STAMP(9);
  }
  __syncthreads();
  RV_STAMP(10);

  int xh[32], xl[32];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 a = *reinterpret_cast<const uint4*>(planes + ((size_t)c * NG + g) * 16);
    const uint4 b = *reinterpret_cast<const uint4*>(planes + ((size_t)(c + 8) * NG + g) * 16);
    xh[4 * c] = (int)a.x; xh[4 * c + 1] = (int)a.y; xh[4 * c + 2] = (int)a.z; xh[4 * c + 3] = (int)a.w;
    xl[4 * c] = (int)b.x; xl[4 * c + 1] = (int)b.y; xl[4 * c + 2] = (int)b.z; xl[4 * c + 3] = (int)b.w;
  }
  const float sx16 = gsx[g];
  const float cq0 = gcq[g * SETS], cq1 = SETS == 2 ? gcq[g * SETS + 1] : 0.f;

  RV_STAMP(3);
  // ---- rows that were copied to shared memory, R at a time: the lanes' partial sums of R rows are
  // reduced together (lanes end up holding different rows), so a row costs 18 / R shuffle-class
  // instructions instead of 10 and the R dot products overlap.
  int bar_i = 0, bar_c = 0;                       // barrier of iteration i = i / ipb, kept without a division
#pragma unroll 1
  for (int i = 0; i < nrows_s; i += R) {
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      acc[r] = 0.f;
      if (i + r < nrows_s) {                      // warp-uniform
        rv_mbar_wait(bar0 + 8 * bar_i, 0, &s_abort, p.status);
        if (++bar_c == ipb) { bar_c = 0; ++bar_i; }
        if (i + r == nrows_s - 1) RV_STAMP(7);
        const unsigned char* rp = srows + (size_t)(rl + (i + r) * RL) * p.rec_bytes;
        uint32_t w[NW];
#pragma unroll
        for (int j = 0; j < J; ++j) {
          const uint4 v = *reinterpret_cast<const uint4*>(rp + woff + j * jstride);
          w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
        }
        const uint32_t scw = SETS == 2 ? *reinterpret_cast<const uint32_t*>(rp + soff)
                                       : (uint32_t)*reinterpret_cast<const uint16_t*>(rp + soff);
        const uint32_t chw = *reinterpret_cast<const uint16_t*>(rp + coff);
        acc[r] = row_value<BITS, SETS>(w, scw, cher_on ? chw : 0u, xh, xl, sx16, cq0, cq1, xc, lane_on);
      }
    }
    const float tot = reduce_rows<R>(acc, lane);  // lane (32 / R) * r holds the total of row r
    if ((lane & (32 / R - 1)) == 0) {
      const int r = lane / (32 / R);
      if (i + r < nrows_s) {
        const int rr = rl + (i + r) * RL;
        float v = tot;
        if (nsl == 1) {
          if (p.accumulate) v += __half2float(p.y[r0 + rr]);
          p.y[r0 + rr] = __float2half_rn(v);
        } else {
          part[rr * nsl + sl] = v;
        }
      }
    }
  }
  // ---- rows read from global memory
  if (D > 0) {
    for (int i = 0; i < nrows_g; i += DG) {
#pragma unroll
      for (int d = 0; d < DG; ++d) {
        const int ii = i + d;
        if (ii < nrows_g) {
          uint32_t w[NW];
#pragma unroll
          for (int j = 0; j < J; ++j) {
            w[4 * j] = wb[d][j].x; w[4 * j + 1] = wb[d][j].y; w[4 * j + 2] = wb[d][j].z; w[4 * j + 3] = wb[d][j].w;
          }
          float acc = row_value<BITS, SETS>(w, sc[d], ch[d], xh, xl, sx16, cq0, cq1, xc, lane_on);
          // the buffers of this row are free: request the row D steps ahead
          const int nn = ii + DG;
          if (nn < nrows_g) {
            const uint8_t* rp = gptr + (size_t)nn * gstep;
            if (lane_on) {
#pragma unroll
              for (int j = 0; j < J; ++j) wb[d][j] = ldg_stream16(rp + woff + j * jstride);
              sc[d] = SETS == 2 ? ldg_stream4(rp + soff) : ldg_stream2(rp + soff);
            }
            if (cher_on) ch[d] = ldg_stream2(rp + coff);
          }
#pragma unroll
          for (int s = 16; s >= 1; s >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, s);
          if (lane == 0) {
            const int rr = rl + (nrows_s + ii) * RL;
            if (nsl == 1) {
              if (p.accumulate) acc += __half2float(p.y[r0 + rr]);
              p.y[r0 + rr] = __float2half_rn(acc);
            } else {
              part[rr * nsl + sl] = acc;
            }
          }
        }
      }
    }
  }
  RV_STAMP(4);
  if (nsl > 1) {
    __syncthreads();
    for (int rr = tid; rr < r1 - r0; rr += NTHR) {
      float acc = p.accumulate ? __half2float(p.y[r0 + rr]) : 0.f;
      for (int s = 0; s < nsl; ++s) acc += part[rr * nsl + s];
      p.y[r0 + rr] = __float2half_rn(acc);
    }
  }
  RV_STAMP(5);
}

// ------------------------------------------------------------------ layout kernels
struct RlayerDev {
  uint8_t* rows; uint16_t* perm; uint16_t* cidx;
  int bits, K, N, C, G, Kc, NG, sets, nsl, gps, row_bytes, srow_bytes, rec_bytes;
};

RlayerDev rl_view(const cq_rlayer* L) {
  RlayerDev d;
  uint8_t* b = (uint8_t*)L->blob;
  d.rows = b + L->off_rows;
  d.perm = (uint16_t*)(b + L->off_perm);
  d.cidx = (uint16_t*)(b + L->off_cidx);
  d.bits = L->bits; d.K = L->K; d.N = L->N; d.C = L->C; d.G = L->G; d.Kc = L->Kc; d.NG = L->NG;
  d.sets = L->sets; d.nsl = L->nsl; d.gps = L->gps; d.row_bytes = L->row_bytes; d.srow_bytes = L->srow_bytes;
  d.rec_bytes = L->rec_bytes;
  return d;
}

// Byte offset (inside the record) of 32-bit word wi of group gg.
__device__ __forceinline__ size_t rl_word_off(const RlayerDev& d, int gg, int wi) {
  const int sl = gg / d.gps, ln = gg - sl * d.gps;
  const int gcount = min(d.gps, d.NG - sl * d.gps);
  return (size_t)sl * d.gps * 16 * d.bits + ((size_t)(wi >> 2) * gcount + ln) * 16 + (wi & 3) * 4;
}
__device__ __forceinline__ __half* rl_scale_ptr(const RlayerDev& d, int n, int gs) {
  return reinterpret_cast<__half*>(d.rows + (size_t)n * d.rec_bytes + d.row_bytes) + gs;
}
__device__ __forceinline__ __half* rl_cherry_ptr(const RlayerDev& d, int n, int c) {
  return reinterpret_cast<__half*>(d.rows + (size_t)n * d.rec_bytes + d.row_bytes + d.srow_bytes) + c;
}

// Where code e (0..127) of a group sits: first word index, per code bit the bit position, and how
// far the word index advances per code bit (1 for the 3-bit bit-plane fields).
__device__ __forceinline__ void rl_code_pos(int bits, int e, int* wi, int* bitpos, int* wstep) {
  if (bits == 4) {
    const int i = e & 7;
    *wi = e >> 3; *wstep = 0;
    const int sh = i < 4 ? 8 * i : 8 * (i - 4) + 4;
    bitpos[0] = sh; bitpos[1] = sh + 1; bitpos[2] = sh + 2; bitpos[3] = sh + 3;
  } else {
    const int s = e >> 5, r = e & 31, f = r >> 2, b = r & 3;
    if (f < 6) {
      *wi = 3 * s + (f >> 1); *wstep = 0;
      const int sh = 8 * b + 4 * (f & 1);
      bitpos[0] = sh; bitpos[1] = sh + 1; bitpos[2] = sh + 2;
    } else {                      // bit planes: bit t of the code lives in word 3s + t
      *wi = 3 * s; *wstep = 1;
      const int sh = 8 * b + (f == 6 ? 3 : 7);
      bitpos[0] = sh; bitpos[1] = sh; bitpos[2] = sh;
    }
  }
}

__device__ __forceinline__ uint32_t rl_read_code(const RlayerDev& d, int n, int kc) {
  const int gg = kc >> 7, e = kc & 127;
  int wi, bp[4], ws;
  rl_code_pos(d.bits, e, &wi, bp, &ws);
  const uint8_t* row = d.rows + (size_t)n * d.rec_bytes;
  uint32_t u = 0;
  for (int t = 0; t < d.bits; ++t) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(row + rl_word_off(d, gg, wi + ws * t));
    u |= ((w >> bp[t]) & 1u) << t;
  }
  return u;
}

// one thread per (row n, group gg, word wi); n fastest so that the reference bytes are read coalesced
__global__ void rl_prepare_codes_kernel(RlayerDev d, const uint8_t* __restrict__ q) {
  const int nw = 4 * d.bits;
  const size_t total = (size_t)d.N * d.NG * nw;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int n = (int)(idx % d.N);
    const size_t rest = idx / d.N;
    const int wi = (int)(rest % nw), gg = (int)(rest / nw);
    uint32_t word = 0;
    for (int e = 0; e < 128; ++e) {
      int cwi, bp[4], ws;
      rl_code_pos(d.bits, e, &cwi, bp, &ws);
      const int kc = gg * 128 + e;
      if (ws == 0) {
        if (cwi != wi || kc >= d.Kc) continue;
        const uint32_t u = cq_ref_code(q, d.bits, kc, n, d.N);
        for (int t = 0; t < d.bits; ++t) word |= ((u >> t) & 1u) << bp[t];
      } else {
        const int t = wi - cwi;
        if (t < 0 || t > 2 || kc >= d.Kc) continue;
        const uint32_t u = cq_ref_code(q, d.bits, kc, n, d.N);
        word |= ((u >> t) & 1u) << bp[t];
      }
    }
    *reinterpret_cast<uint32_t*>(d.rows + (size_t)n * d.rec_bytes + rl_word_off(d, gg, wi)) = word;
  }
}

// scales (per 128-column group and set), cherry values, column permutation and cherry list
__global__ void rl_prepare_rest_kernel(RlayerDev d, const __half* __restrict__ scales, const __half* __restrict__ cw,
                                       const int16_t* __restrict__ ci) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int ngr = (d.Kc + d.G - 1) / d.G;            // scale rows of the reference
  const int spr = d.srow_bytes / 2;                  // scale slots per row, padding included
  for (size_t idx = t0; idx < (size_t)d.N * spr; idx += stride) {
    const int n = (int)(idx % d.N);
    const int gs = (int)(idx / d.N);
    const int kc = (gs / d.sets) * 128 + (gs % d.sets) * 64;
    const int gi = kc / d.G;
    const bool real = gs < d.NG * d.sets && kc < d.Kc && gi < ngr;
    *rl_scale_ptr(d, n, gs) = real ? scales[(size_t)gi * d.N + n] : __float2half(0.f);
  }
  for (size_t idx = t0; idx < (size_t)d.N * d.C; idx += stride) {
    const int n = (int)(idx % d.N), c = (int)(idx / d.N);
    *rl_cherry_ptr(d, n, c) = cw[(size_t)c * d.N + n];
  }
  for (size_t idx = t0; idx < (size_t)d.NG * 128; idx += stride) {
    const int kc = (int)idx;
    uint32_t col = (uint32_t)d.K;                  // padding columns read the kernel's zero slot
    if (kc < d.Kc) {
      // number of cherry columns at or before the kc-th normal column (the reference's upper-bound
      // search, csrc/quant_cuda_kernel.cu:785-795)
      int low = 0, high = d.C;
      while (low < high) {
        const int mid = (low + high) >> 1;
        if ((int)(uint16_t)ci[mid] - mid <= kc) low = mid + 1; else high = mid;
      }
      col = (uint32_t)(kc + low);
    }
    d.perm[kc] = (uint16_t)col;
  }
  for (size_t idx = t0; idx < (size_t)d.C; idx += stride) d.cidx[idx] = (uint16_t)ci[idx];
}

__global__ void rl_unprepare_kernel(RlayerDev d, uint8_t* __restrict__ q, __half* __restrict__ scales,
                                    __half* __restrict__ cw, int16_t* __restrict__ ci) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  // codes: one thread per 8 compact columns of a row
  const size_t no = (size_t)d.N * (d.Kc / 8);
  for (size_t idx = t0; idx < no; idx += stride) {
    const int n = (int)(idx % d.N), o = (int)(idx / d.N);
    uint32_t u[8];
    for (int i = 0; i < 8; ++i) u[i] = rl_read_code(d, n, 8 * o + i);
    if (d.bits == 4) {
      for (int i = 0; i < 4; ++i) q[(size_t)(4 * o + i) * d.N + n] = (uint8_t)(u[2 * i] | (u[2 * i + 1] << 4));
    } else {
      uint32_t w = 0;
      for (int i = 0; i < 8; ++i) w |= u[i] << (3 * i);
      for (int i = 0; i < 3; ++i) q[(size_t)(3 * o + i) * d.N + n] = (uint8_t)(w >> (8 * i));
    }
  }
  const int ngr = (d.Kc + d.G - 1) / d.G;
  for (size_t idx = t0; idx < (size_t)d.N * ngr; idx += stride) {
    const int n = (int)(idx % d.N), gi = (int)(idx / d.N);
    const int kc = gi * d.G;
    scales[(size_t)gi * d.N + n] = *rl_scale_ptr(d, n, (kc >> 7) * d.sets + ((kc >> 6) & (d.sets - 1)));
  }
  for (size_t idx = t0; idx < (size_t)d.N * d.C; idx += stride) {
    const int n = (int)(idx % d.N), c = (int)(idx / d.N);
    cw[(size_t)c * d.N + n] = *rl_cherry_ptr(d, n, c);
  }
  for (size_t idx = t0; idx < (size_t)d.C; idx += stride) ci[idx] = (int16_t)d.cidx[idx];
}

// ------------------------------------------------------------------ host side
typedef void (*RowvecFn)(const RowvecParams);

struct RvDevice { int sms = 0, max_smem = 0; bool ok = false; };
RvDevice rv_device(int dev) {
  static RvDevice cache[64];
  if (dev < 0 || dev >= 64) return RvDevice();
  if (!cache[dev].ok) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return RvDevice();
    cache[dev].sms = prop.multiProcessorCount;
    cache[dev].max_smem = (int)prop.sharedMemPerBlockOptin;
    cache[dev].ok = true;
  }
  return cache[dev];
}

inline int rv_align(int v, int a) { return (v + a - 1) / a * a; }

template <int W, int D, int R>
RowvecFn rv_pick(int bits, int sets) {
  if (bits == 4) return sets == 1 ? cq_rowvec_kernel<4, 1, W, D, R> : cq_rowvec_kernel<4, 2, W, D, R>;
  return sets == 1 ? cq_rowvec_kernel<3, 1, W, D, R> : cq_rowvec_kernel<3, 2, W, D, R>;
}

// One launch; `fn`'s warp count is W and its global-memory pipeline depth D (0: none).
// smem_kb caps the shared memory a CTA takes (0: all of it).
int rv_launch(RowvecFn fn, int W, int D, int pre_pct, int smem_kb, const cq_rlayer* L, const __half* x, __half* y,
              int accumulate, uint32_t* status, cudaStream_t st) {
  int dev = 0;
  CQ_CUDA_TRY(cudaGetDevice(&dev));
  const RvDevice di = rv_device(dev);
  if (!di.ok) return CQ_ERR_NO_DEVICE;
  if (L->nsl > W) return CQ_ERR_UNSUPPORTED;
  int grid = di.sms;
  const int RL = W / L->nsl;
  const int want = (L->N + RL - 1) / RL;
  if (grid > want) grid = want;
  if (grid < 1) grid = 1;
  const int rows_max = (L->N + grid - 1) / grid + 1;

  RowvecParams p;
  const uint8_t* blob = (const uint8_t*)L->blob;
  p.rows = blob + L->off_rows;
  p.perm = (const uint16_t*)(blob + L->off_perm);
  p.cidx = (const uint16_t*)(blob + L->off_cidx);
  p.x = x; p.y = y; p.status = status;
  p.K = L->K; p.N = L->N; p.C = L->C; p.NG = L->NG; p.nsl = L->nsl; p.gps = L->gps; p.cps = L->cps;
  p.accumulate = accumulate; p.row_bytes = L->row_bytes; p.srow_bytes = L->srow_bytes; p.rec_bytes = L->rec_bytes;
#ifdef CQ_ROWVEC_TRACE
  static int launch_no = 0;
  p.trace_launch = launch_no++;
#endif
  int off = rv_align((L->K + 8) * 2, 16);
  p.off_planes = off; off += 256 * L->NG;
  p.off_sx = off; off = rv_align(off + (1 + L->sets) * 4 * L->NG, 16);
  p.off_part = off; off = rv_align(off + (L->nsl > 1 ? rows_max * L->nsl * 4 : 0), 16);
  p.off_bar = off; off = rv_align(off + RV_NBAR * 8, 128);
  p.off_rows = off;
  int budget = di.max_smem - 64;            // the kernel also has a small static allocation
  if (smem_kb > 0 && smem_kb * 1024 < budget) budget = smem_kb * 1024;
  int smem_rows = (budget - off) / L->rec_bytes;
  if (smem_rows < 0) smem_rows = 0;
  if (smem_rows > rows_max) smem_rows = rows_max;
  if (D == 0 && smem_rows < rows_max) return CQ_ERR_TOO_LARGE;
  p.smem_rows = smem_rows;
  p.rows_q = L->N / grid; p.rows_r = L->N % grid;
  p.pre_pct = pre_pct % 1000;
  p.l2_prefetch = pre_pct / 1000;
  const int smem = off + smem_rows * L->rec_bytes;
  if (smem > di.max_smem) return CQ_ERR_TOO_LARGE;
  CQ_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(W * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, fn, p));
  return CQ_OK;
}
}  // namespace

#ifndef CQ_ROWVEC_W
#define CQ_ROWVEC_W 12
#define CQ_ROWVEC_D 2
#define CQ_ROWVEC_PRE 60
#define CQ_ROWVEC_R 4
#define CQ_ROWVEC_PF 0
#endif

extern "C" int cq_rlayer_init(cq_rlayer* L, int bits, int K, int N, int C, int G, void* blob) {
  if (!L) return CQ_ERR_BAD_ARG;
  if (bits != 3 && bits != 4) return CQ_ERR_BAD_BITS;
  if (G == -1) G = K;
  if (!(G == 64 || (G > 0 && G % 128 == 0))) return CQ_ERR_BAD_GROUP;
  if (bits == 4 && G < 128) return CQ_ERR_BAD_GROUP;
  if (K <= 0 || N <= 0 || C < 0 || K % 8 || C % 8 || C >= K || K > 65534) return CQ_ERR_BAD_SHAPE;
  L->bits = bits; L->K = K; L->N = N; L->C = C; L->G = G;
  L->Kc = K - C;
  L->NG = (L->Kc + 127) / 128;
  L->sets = G == 64 ? 2 : 1;
  L->nsl = (L->NG + 31) / 32;
  L->gps = (L->NG + L->nsl - 1) / L->nsl;
  L->cps = (C + L->nsl - 1) / L->nsl;
  if (L->cps > 32) return CQ_ERR_UNSUPPORTED;      // more than 32 cherry columns per 4096 columns
  L->row_bytes = L->NG * 16 * bits;
  L->srow_bytes = (L->NG * L->sets * 2 + 15) / 16 * 16;
  L->rec_bytes = L->row_bytes + L->srow_bytes + C * 2;
  uint64_t off = 0;
  L->off_rows = off;   off += (uint64_t)N * L->rec_bytes;           off = (off + 255) / 256 * 256;
  L->off_perm = off;   off += (uint64_t)L->NG * 128 * 2;            off = (off + 255) / 256 * 256;
  L->off_cidx = off;   off += (uint64_t)(C > 0 ? C : 8) * 2;        off = (off + 255) / 256 * 256;
  L->blob_bytes = off;
  L->blob = blob;
  return CQ_OK;
}

extern "C" int cq_rlayer_prepare(const cq_rlayer* L, const uint8_t* qweight, const void* scales, const void* cherry_weight,
                                 const int16_t* cherry_indices, cq_stream_t stream) {
  if (!L || !L->blob || !qweight || !scales) return CQ_ERR_BAD_ARG;
  if (L->C > 0 && (!cherry_weight || !cherry_indices)) return CQ_ERR_BAD_ARG;
  if ((uintptr_t)L->blob & 255) return CQ_ERR_BAD_ARG;
  const RlayerDev d = rl_view(L);
  cudaStream_t st = (cudaStream_t)stream;
  rl_prepare_codes_kernel<<<2048, 256, 0, st>>>(d, qweight);
  CQ_CUDA_TRY(cudaGetLastError());
  rl_prepare_rest_kernel<<<1024, 256, 0, st>>>(d, (const __half*)scales, (const __half*)cherry_weight, cherry_indices);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}

extern "C" int cq_rlayer_unprepare(const cq_rlayer* L, uint8_t* qweight, void* scales, void* cherry_weight,
                                   int16_t* cherry_indices, cq_stream_t stream) {
  if (!L || !L->blob || !qweight || !scales) return CQ_ERR_BAD_ARG;
  if (L->C > 0 && (!cherry_weight || !cherry_indices)) return CQ_ERR_BAD_ARG;
  const RlayerDev d = rl_view(L);
  rl_unprepare_kernel<<<2048, 256, 0, (cudaStream_t)stream>>>(d, qweight, (__half*)scales, (__half*)cherry_weight,
                                                              cherry_indices);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}

extern "C" int cq_rlayer_matvec(const cq_rlayer* L, const void* x, void* y, int accumulate, uint32_t* status_word,
                                cq_stream_t stream) {
  if (!L || !L->blob || !x || !y) return CQ_ERR_BAD_ARG;
  if (((uintptr_t)x & 1) || ((uintptr_t)y & 1)) return CQ_ERR_BAD_ARG;
  return rv_launch(rv_pick<CQ_ROWVEC_W, CQ_ROWVEC_D, CQ_ROWVEC_R>(L->bits, L->sets), CQ_ROWVEC_W, CQ_ROWVEC_D, CQ_ROWVEC_PRE + 1000 * CQ_ROWVEC_PF, 0, L,
                   (const __half*)x, (__half*)y, accumulate, status_word, (cudaStream_t)stream);
}

#ifdef CQ_ROWVEC_SWEEP
// Tuning build only (not part of the library): a table of kernel shapes behind one entry point.
#define RV_CASE(id, W, D, R, SMEM_KB, PRE, PF) \
  case id: return rv_launch(rv_pick<W, D, R>(L->bits, L->sets), W, D, PRE + 1000 * PF, SMEM_KB, L, (const __half*)x, (__half*)y, accumulate, status_word, (cudaStream_t)stream);
extern "C" int cq_rlayer_matvec_variant(int variant, const cq_rlayer* L, const void* x, void* y, int accumulate,
                                        uint32_t* status_word, cq_stream_t stream) {
  switch (variant) {
    CQ_ROWVEC_SWEEP
    default: return CQ_ERR_UNSUPPORTED;
  }
}
#ifdef CQ_ROWVEC_TRACE
extern "C" int cq_rv_set_trace(void* device_buffer) {
  unsigned long long* ptr = (unsigned long long*)device_buffer;
  CQ_CUDA_TRY(cudaMemcpyToSymbol(cq_rv_trace, &ptr, sizeof(ptr)));
  return CQ_OK;
}
#endif
#endif
