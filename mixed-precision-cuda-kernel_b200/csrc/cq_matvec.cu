// Decode matvec of one prepared CherryQ layer for 1..16 activation rows:
//   y[m, n] (+)= sum_k' (u[k', n] - off) * s[group(k'), n] * x[m, orig(k')]
//              + sum_c  cherry_weight[c, n] * x[m, idx[c]]
// which is what the reference kernels compute (csrc/quant_cuda_kernel.cu:718-835
// for 4-bit, :558-672 for 3-bit, :316-438 for 3-bit with 64-wide groups, of the
// reference project), with fp32 accumulation and one fp16 store per output.
//
// Shape of the kernel (one persistent CTA per SM, HBM-bandwidth bound):
//  * The layer's stream (see cq_common.cuh) is a flat sequence of granules
//    (16 rows x 128 compact columns).  CTA c owns the contiguous granule range
//    [T*c/grid, T*(c+1)/grid): an equal byte share whatever N and K are.
//  * A producer warp moves the range into a shared-memory ring with 1-D bulk
//    async copies (cp.async.bulk + mbarrier transaction counts), 2 * NCW
//    granules per copy.  It starts before the kernel waits for the previous kernel
//    in the stream (programmatic dependent launch): weights never depend on it.
//  * NCW consumer warps take the granules of a copy two each.  A lane reads
//    its 32 (4-bit) or 24 (3-bit) bytes and turns them into the A fragments of the integer
//    tensor-core instruction mma.sync.m16n8k32 (u8 x s8 -> s32) with one or two logic
//    operations per four codes (byte masks; no conversion, no arithmetic per weight).
//    The activations are the B operand: while they are staged (once per launch, in compact
//    column order) every granule's 128 values of a row are scaled to 15-bit integers
//    q = 128 hi + lo and stored as two signed bytes, which occupy two of the MMA's eight B
//    columns, so one MMA yields sum(u hi) and sum(u lo) exactly.  Per granule and group:
//        y += s * (sx * (128 sum(u hi) + sum(u lo)) - off * sx * sum(q))
//    with sx the activation step of that granule; the last term is prepared while staging.
//    The cherry columns stay fp16 x fp16 on mma.sync.m16n8k16.
//  * A range is walked from its last sub-tile to its first.  A sub-tile cut by a
//    range boundary is finished by the CTA that holds its end: CTAs holding an
//    earlier part post their fp32 partial to global scratch early in their walk,
//    the finishing CTA adds the partials in a fixed order late in its walk.  All
//    sums are therefore deterministic.  Every wait is bounded; running out sets
//    a bit in the status word instead of hanging.
#include <cstdlib>
#include <mutex>

#include "cq_common.cuh"

#ifdef CQ_MATVEC_TRACE
unsigned long long* cq_g_timeline = nullptr;   // tracing buffer of instrumented builds, see cq_trace_set_timeline
#endif

namespace {

constexpr uint32_t WAIT_LIMIT = 1u << 22;

struct MatvecParams {
  const uint8_t* stream;
  const uint8_t* cstream;
  const uint16_t* cidx;
  const uint32_t* osh;
  const __half* x;
  __half* y;
  float* partial;      // [grid][256]
  uint32_t* flag;      // [grid]
  uint32_t* status;    // may be null
  unsigned long long* timeline;  // may be null: [grid][64] %globaltimer stamps (tracing)
  int M, K, N, C, Cp, Kp, n_gran, n_sub, gran_bytes, cher_bytes;
  int ldx, ldy, accumulate;
  uint32_t T;          // total granules
  int stages, nslot, max_cher, inflight;
  // shared-memory offsets
  int off_ring, off_cher, off_zero, off_sched, off_xb, off_xq, off_xc, off_slot, off_pf, off_bar;
  int xb_gran;         // bytes of quantised activations per granule: 2 planes x 2M columns x 64 B
  int xc_stride;       // halves per cherry-activation row (Cp + 8)
};

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: gives up after WAIT_LIMIT polls (or at once when the CTA already
// gave up somewhere), records the failure and lets the caller carry on.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                            uint32_t* status) {
  // bounded in polls and in time (about one second of the device's nanosecond timer)
  const uint32_t limit = *abort_flag ? 1u : WAIT_LIMIT;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status);
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
template <int NCONS>
__device__ __forceinline__ void bar_consumers() {
  asm volatile("bar.sync 1, %0;" ::"n"(NCONS) : "memory");
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// D = A (16 x 32 unsigned bytes) . B (32 x 8 signed bytes) + C, 32-bit integers
__device__ __forceinline__ void imma16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1, int c0, int c1, int c2, int c3) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
}

__device__ __forceinline__ void stamp(const MatvecParams& p, int slot) {
  if (p.timeline) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.timeline[(size_t)blockIdx.x * 64 + slot] = t;
  }
}

// ------------------------------------------------------------------ decode
// Activations are quantised per granule to integers |q| <= QMAX = 127 * 128 and split as
// q = 128 hi + lo with hi in [-127, 127], lo in [-64, 63].
constexpr float QMAX = 16256.f;
template <int BITS> struct CodeOffset;
template <> struct CodeOffset<4> { static constexpr float OFF = 7.5f; };
template <> struct CodeOffset<3> { static constexpr float OFF = 3.5f; };

// Fragment registers j = 0..7 of one row (four codes each, one per byte) from the row's words.
__device__ __forceinline__ void regs4(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t* R) {
  constexpr uint32_t M4 = 0x0F0F0F0Fu;
  R[0] = w0 & M4; R[1] = (w0 >> 4) & M4;
  R[2] = w1 & M4; R[3] = (w1 >> 4) & M4;
  R[4] = w2 & M4; R[5] = (w2 >> 4) & M4;
  R[6] = w3 & M4; R[7] = (w3 >> 4) & M4;
}
__device__ __forceinline__ void regs3(uint32_t a, uint32_t b, uint32_t c, uint32_t* R) {
  constexpr uint32_t M3 = 0x07070707u;
  R[0] = a & M3; R[1] = (a >> 3) & M3;
  R[2] = b & M3; R[3] = (b >> 3) & M3;
  R[4] = c & M3; R[5] = (c >> 3) & M3;
  R[6] = ((a >> 6) & 0x03030303u) | ((b >> 4) & 0x04040404u);
  R[7] = ((c >> 6) & 0x03030303u) | ((b >> 5) & 0x04040404u);
}

// Geometry of piece i of a CTA's range (pieces = sub-tiles, walked from the last to the first).
struct Piece {
  uint32_t j, sub0, start, end;   // sub-tile, its first granule, first / past-last granule of the piece
};
__device__ __forceinline__ Piece piece_of(uint32_t i, uint32_t j_hi, uint32_t NG, uint32_t ga, uint32_t gb) {
  Piece q;
  q.j = j_hi - i;
  q.sub0 = q.j * NG;
  q.start = max(ga, q.sub0);
  q.end = min(gb, q.sub0 + NG);
  return q;
}

// The packed words of one granule that one lane needs, loaded one ring stage ahead of their use.
template <int BITS, int SETS> struct Raw;
template <int SETS> struct Raw<4, SETS> { uint4 a, b; uint32_t sc[SETS]; };
template <int SETS> struct Raw<3, SETS> { uint4 a; uint2 b; uint32_t sc[SETS]; };

// MB = activation tiles of four rows (two B columns per row); MAXR = register cap per thread
// (SMALL_NCW / LARGE_NCW on the host side).
template <int BITS, int SETS, int MB, int NCW, int MAXR>
__global__ void __launch_bounds__((NCW + 1) * 32) __maxnreg__(MAXR) cq_matvec_kernel(const MatvecParams p) {
  constexpr int NCONS = NCW * 32;
  constexpr uint32_t CH = 2 * NCW;        // granules per ring stage: a pair per consumer warp
  constexpr int MBH = (MB + 1) / 2;       // fp16 MMA tiles of eight activation rows (cherry columns)
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t grid = gridDim.x, cta = blockIdx.x;
  const uint32_t ga = (uint32_t)(((uint64_t)p.T * cta) / grid);
  const uint32_t gb = (uint32_t)(((uint64_t)p.T * (cta + 1)) / grid);
  const uint32_t NG = (uint32_t)p.n_gran;
  const uint32_t GB = (uint32_t)p.gran_bytes;
  const uint32_t total = gb - ga;

  const uint32_t bar_base = smem_u32(smem + p.off_bar);
  const uint32_t S = (uint32_t)p.stages;
  // barriers: full[s] at bar_base + 8 s, empty[s] at + 8 (S + s), cherry at + 16 S, partial prefetch at + 16 S + 8
  if (tid == 0) {
    stamp(p, 0);
    s_abort = 0;
    for (uint32_t s = 0; s < S; ++s) {
      mbar_init(bar_base + 8 * s, 1);
      mbar_init(bar_base + 8 * (S + s), NCW);
    }
    mbar_init(bar_base + 16 * S, 1);
    mbar_init(bar_base + 16 * S + 8, 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  if (tid == 0) stamp(p, 1);
  // Let the next kernel in the stream start its own prologue and weight prefetch.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (ga >= gb) return;  // (host launches grid <= T, so this does not happen)

  const uint32_t j_hi = (gb - 1) / NG, j_lo = ga / NG;
  const uint32_t npieces = j_hi - j_lo + 1;
  const uint32_t jc_lo = (ga + NG - 1) / NG;           // first sub-tile whose start is in range
  const int ncher = (p.Cp > 0 && j_hi >= jc_lo) ? (int)(j_hi - jc_lo + 1) : 0;

  // ------------------------------------------------------------------ producer
  // The CTA's granules, in walking order, form a sequence of `total` positions.  Ring stage
  // (i mod S) holds positions [i * CH, (i + 1) * CH): position q sits at slot q mod CH of it
  // and belongs to consumer warp (q mod CH) / 2.  A stage is filled by one bulk copy per piece it
  // touches (granules of a piece are contiguous in memory).
  if (warp == NCW) {
    if (lane == 0) {
      if (ncher > 0) {
        const uint32_t bytes = (uint32_t)ncher * (uint32_t)p.cher_bytes;
        mbar_expect_tx(bar_base + 16 * S, bytes);
        bulk_g2s(smem_u32(smem + p.off_cher), p.cstream + (size_t)jc_lo * p.cher_bytes, bytes,
                 bar_base + 16 * S);
      }
      const uint32_t ring = smem_u32(smem + p.off_ring);
      uint32_t stage = 0, phase = 1;   // empty barriers: the first pass over the ring needs no wait
      bool first_pass = true;
      stamp(p, 8);
      uint32_t pi = 0;
      Piece pc = piece_of(0, j_hi, NG, ga, gb);
      uint32_t src = pc.start;           // next granule to copy
      const uint32_t INFL = (uint32_t)p.inflight;
      uint32_t k = 0;                    // stage counter
      for (uint32_t q0 = 0; q0 < total; q0 += CH, ++k) {
        const uint32_t len = min(CH, total - q0);
        if (!first_pass) mbar_wait(bar_base + 8 * (S + stage), phase, &s_abort, p.status);
        // Pace the copies: at most INFL stages are outstanding, so that stages land in order and the
        // first one is usable early (the memory system interleaves everything that is in flight).
        // (only while the ring is deeper than that: otherwise the slot wait above paces already, and the
        // barrier of stage k - INFL may have been re-armed)
        if (INFL < S && k >= INFL) mbar_wait(bar_base + 8 * ((k - INFL) % S), ((k - INFL) / S) & 1, &s_abort, p.status);
        mbar_expect_tx(bar_base + 8 * stage, len * GB);
        uint32_t dst = ring + stage * CH * GB, left = len;
        while (left > 0) {
          if (src == pc.end) {
            pc = piece_of(++pi, j_hi, NG, ga, gb);
            src = pc.start;
          }
          const uint32_t run = min(left, pc.end - src);
          bulk_g2s(dst, p.stream + (size_t)src * GB, run * GB, bar_base + 8 * stage);
          dst += run * GB;
          src += run;
          left -= run;
        }
        if (++stage == S) { stage = 0; phase ^= 1; first_pass = false; }
      }
      stamp(p, 9);
    }
    // The sub-tile at the head of this range may have been started by earlier CTAs, which posted
    // their partials early in their walk.  Fetch them now (this warp is idle) so that the
    // consumers find the sum in shared memory when they finish the sub-tile.  The scratch may
    // still hold the previous launch's flags until that launch has completed: wait for it first.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
      float* pf = reinterpret_cast<float*>(smem + p.off_pf);
      const uint32_t s0g = j_lo * NG;
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
      if (ga > s0g && gb >= s0g + NG) {
        const uint32_t c_first = (uint32_t)((((uint64_t)s0g + 1) * grid - 1) / p.T);
        for (uint32_t c = c_first; c < cta; ++c) {
          bool ok = false;
          const uint32_t limit = s_abort ? 1u : WAIT_LIMIT;
          for (uint32_t it = 0; it < limit; ++it) {
            if (ld_acquire(p.flag + c) != 0) { ok = true; break; }
            __nanosleep(64);
          }
          if (!ok) {
            s_abort = 1;
            if (p.status) atomicOr(p.status, 2u);
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] += __ldcg(p.partial + (size_t)c * 256 + e * 32 + lane);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) pf[e * 32 + lane] = v[e];
      mbar_arrive(bar_base + 16 * S + 8);   // release: the consumers wait on this barrier
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  // Layer constants first (they do not depend on the previous kernel).  The index tables (sorted
  // cherry columns; per octet of compact columns, how far its first and last column are shifted in
  // the original row, see cq_common.cuh) are read straight from global memory into registers: the
  // entries of a thread's first items are requested here, so that they are at hand when the
  // dependency wait returns and the activation loads can be issued at once.
  __half* xc = reinterpret_cast<__half*>(smem + p.off_xc);
  const int noct = p.Kp >> 3;
  constexpr int XCU = 2;      // cherry activations a thread fetches ahead
  constexpr int U = 2;        // octets of compact columns a thread stages per round
  const int nitem = noct * p.M;
  uint32_t sh_first[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int it = u * NCONS + tid;
    sh_first[u] = it < nitem ? __ldg(p.osh + (p.M == 1 ? it : it % noct)) : 0xFFFFFFFFu;
  }
  uint32_t cher_col[XCU];
#pragma unroll
  for (int u = 0; u < XCU; ++u) {
    const int idx = tid + u * NCONS;
    cher_col[u] = idx < p.M * p.Cp ? (uint32_t)__ldg(p.cidx + idx % p.Cp) : (uint32_t)CQ_PAD_COL;
  }
  // {step, offset terms} of activation rows that do not exist must read as zero
  for (int i = tid; i < (int)NG * 4 * MB * 4; i += NCONS) reinterpret_cast<float*>(smem + p.off_xq)[i] = 0.f;
  {
    // Schedule: for every position of the CTA's sequence, which granule of its sub-tile it is (low 10
    // bits) and which piece it belongs to.  Piece 0 is the tail of the range (possibly a cut
    // sub-tile), the pieces after it are whole sub-tiles, the last one may be cut at its start.
    uint32_t* sched = reinterpret_cast<uint32_t*>(smem + p.off_sched);
    const Piece p0 = piece_of(0, j_hi, NG, ga, gb);
    const uint32_t len0 = p0.end - p0.start;
    const uint32_t padded = (total + CH - 1) / CH * CH;
    for (uint32_t q = (uint32_t)tid; q < padded; q += NCONS) {
      const uint32_t qq = q < total ? q : total - 1;
      uint32_t pi, gi;
      if (qq < len0) {
        pi = 0;
        gi = p0.start - p0.sub0 + qq;
      } else {
        const uint32_t rest = qq - len0;
        pi = 1 + rest / NG;
        const Piece pq = piece_of(pi, j_hi, NG, ga, gb);
        gi = pq.start - pq.sub0 + (rest - (pi - 1) * NG);
      }
      sched[q] = gi | (pi << 10);
    }
  }
  if (tid < 4) reinterpret_cast<uint32_t*>(smem + p.off_zero)[tid] = 0u;
  bar_consumers<NCONS>();       // (the zero fill above must not overtake the staging stores below)
  if (tid == 0) stamp(p, 2);

  // Everything below may read what the previous kernel in the stream wrote.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (tid == 0) stamp(p, 3);

  // Activations of the cherry columns: issue the loads now, store them after the main gather,
  // so that both cost one trip to L2 together.
  __half xcv[XCU];
#pragma unroll
  for (int u = 0; u < XCU; ++u) {
    const int idx = tid + u * NCONS;
    xcv[u] = __float2half(0.f);
    if (cher_col[u] != CQ_PAD_COL) xcv[u] = __ldg(p.x + (size_t)(idx / p.Cp) * p.ldx + cher_col[u]);
  }
  {
    // Compact columns, 8 at a time (zero past K').  The 16 octets of one granule of one row sit
    // in 16 neighbouring lanes: they agree on the granule's largest magnitude, quantise, and
    // add up the integers per group.
    for (int base = 0; base < nitem; base += NCONS * U) {
      uint32_t v[U][4];
      int mrow[U], oct[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int it = base + u * NCONS + tid;
        mrow[u] = -1;
        if (base + u * NCONS + (tid & ~31) >= nitem) continue;   // the whole warp is past the last item
        oct[u] = 0;
        v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0u;
        if (it < nitem) {
          const int m = (p.M == 1) ? 0 : it / noct;
          const int o = it - m * noct;
          const int k0 = 8 * o;
          mrow[u] = m;
          oct[u] = o;
          const uint32_t sh = (base == 0) ? sh_first[u] : __ldg(p.osh + o);
          if (sh != 0xFFFFFFFFu) {
            const int lo0 = (int)(sh & 0xFFFFu), lo7 = (int)(sh >> 16);
            const __half* xr = p.x + (size_t)m * p.ldx;
            if (lo7 == lo0) {
              const int src = k0 + lo0;
              if ((src & 1) == 0 && (((uintptr_t)xr) & 3) == 0) {
                const uint32_t* s32 = reinterpret_cast<const uint32_t*>(xr + src);
#pragma unroll
                for (int i = 0; i < 4; ++i) v[u][i] = __ldg(s32 + i);
              } else {
                const unsigned short* s16 = reinterpret_cast<const unsigned short*>(xr + src);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  v[u][i] = (uint32_t)__ldg(s16 + 2 * i) | ((uint32_t)__ldg(s16 + 2 * i + 1) << 16);
              }
            } else {
              // cherry columns fall inside this octet: the shift grows from lo0 to lo7 along it
              unsigned short h[8];
              int sft = lo0;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                while (sft < lo7 && (int)__ldg(p.cidx + sft) - sft <= k0 + i) ++sft;
                h[i] = __ldg(reinterpret_cast<const unsigned short*>(xr + k0 + i + sft));
              }
#pragma unroll
              for (int i = 0; i < 4; ++i) v[u][i] = (uint32_t)h[2 * i] | ((uint32_t)h[2 * i + 1] << 16);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (base + u * NCONS + (tid & ~31) >= nitem) continue;   // (warp-uniform: the shuffles below stay whole)
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 t2 = __half22float2(*reinterpret_cast<const __half2*>(&v[u][i]));
          f[2 * i] = t2.x;
          f[2 * i + 1] = t2.y;
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
#pragma unroll
        for (int d = 1; d < 16; d <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
        // (an infinite or NaN activation makes the step infinite or NaN: the outputs of the rows it
        // feeds come out NaN, as they do in the reference)
        // (reciprocal and products instead of two divisions: each is one correctly rounded operation)
        const float inv = amax > 0.f ? QMAX * __frcp_rn(amax) : 0.f;
        const float sx = amax * (1.f / QMAX);
        int q[8], qsum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          q[i] = __float2int_rn(f[i] * inv);
          qsum += q[i];
        }
#pragma unroll
        for (int d = 1; d < 16 / SETS; d <<= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, d);
        if (mrow[u] >= 0) {
          uint32_t hw[2] = {0u, 0u}, lw[2] = {0u, 0u};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int hi = (q[i] + 64) >> 7;
            const int lo = q[i] - (hi << 7);
            hw[i >> 2] |= ((uint32_t)hi & 0xFFu) << (8 * (i & 3));
            lw[i >> 2] |= ((uint32_t)lo & 0xFFu) << (8 * (i & 3));
          }
          // columns kk = 8 oo .. 8 oo + 7 of the granule: plane kk >> 6, lane column c = (kk >> 2) & 3
          // (two of them), bytes ((kk >> 4) & 3) * 4 + i of the lane's 16
          const int gi = oct[u] >> 4, oo = oct[u] & 15;
          uint8_t* dst = smem + p.off_xb + (size_t)gi * p.xb_gran + (oo >> 3) * (p.M * 128) +
                         (2 * mrow[u]) * 64 + (2 * (oo & 1)) * 16 + ((oo >> 1) & 3) * 4;
          *reinterpret_cast<uint32_t*>(dst) = hw[0];
          *reinterpret_cast<uint32_t*>(dst + 16) = hw[1];
          *reinterpret_cast<uint32_t*>(dst + 64) = lw[0];
          *reinterpret_cast<uint32_t*>(dst + 80) = lw[1];
          if ((oo & (16 / SETS - 1)) == 0) {
            float* xq = reinterpret_cast<float*>(smem + p.off_xq) + ((size_t)gi * 4 * MB + mrow[u]) * 4;
            const float nc = (-CodeOffset<BITS>::OFF * (float)qsum) * sx;
            if (oo == 0) { xq[0] = sx; xq[1] = nc; } else { xq[2] = nc; }
          }
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < XCU; ++u) {
    const int idx = tid + u * NCONS;
    if (idx < p.M * p.Cp) {
      const int m = idx / p.Cp, c = idx - m * p.Cp;
      xc[m * p.xc_stride + c] = xcv[u];
    }
  }
  for (int idx = tid + XCU * NCONS; idx < p.M * p.Cp; idx += NCONS) {
    const int m = idx / p.Cp, c = idx - m * p.Cp;
    const uint32_t o = __ldg(p.cidx + c);
    xc[m * p.xc_stride + c] = (o != CQ_PAD_COL) ? p.x[(size_t)m * p.ldx + o] : __float2half(0.f);
  }
  bar_consumers<NCONS>();
  if (tid == 0) stamp(p, 4);

  const int g = lane >> 2, t = lane & 3;
  float* slots = reinterpret_cast<float*>(smem + p.off_slot);   // [slot][warp][m][16 rows]

  // integer path: tot[b][0] = (row g, activation row 4b + t), tot[b][1] = (row g + 8, same)
  float tot[MB][2];
#pragma unroll
  for (int b = 0; b < MB; ++b) tot[b][0] = tot[b][1] = 0.f;
  // cherry path (fp16 MMA fragment order): ctot[b][0..3] = (row g, activation rows 8b + 2t, + 1), (row g + 8, same)
  float ctot[MBH][4];
#pragma unroll
  for (int b = 0; b < MBH; ++b) ctot[b][0] = ctot[b][1] = ctot[b][2] = ctot[b][3] = 0.f;
  bool did_cher = false;

  // Shared-memory byte offsets (relative to `smem`) this lane reads in every granule.
  // B column n = lane >> 2 of activation tile b is byte plane (n & 1: hi, lo) of activation row
  // 4b + (n >> 1); columns of rows that do not exist are fed zeros.
  const uint32_t xb_off = (uint32_t)p.off_xb + (uint32_t)lane * 16u;
  const uint32_t xb_plane = (uint32_t)p.M * 128u;
  const uint32_t xq_off = (uint32_t)p.off_xq + (uint32_t)t * 16u;
  uint32_t xc_off[MBH];
#pragma unroll
  for (int b = 0; b < MBH; ++b) {
    const int m = (8 * b + g) % p.M;
    xc_off[b] = (uint32_t)p.off_xc + (uint32_t)(m * p.xc_stride + 2 * t) * 2u;
  }
  const uint32_t ring_off = (uint32_t)p.off_ring + 2u * (uint32_t)warp * GB;  // this warp's pair of slots in stage 0
  // B column lane >> 2 of tile b: where this lane's 16 bytes of plane 0 are, how far plane 1 and the
  // next granule are; a column past the last activation row reads the zero block with strides 0
  uint32_t xcol_off[MB], xcol_gran[MB], xcol_plane[MB];
#pragma unroll
  for (int b = 0; b < MB; ++b) {
    const bool has = 8 * b + g < 2 * p.M;
    xcol_off[b] = has ? xb_off + b * 512 : (uint32_t)p.off_zero;
    xcol_gran[b] = has ? (uint32_t)p.xb_gran : 0u;
    xcol_plane[b] = has ? xb_plane : 0u;
  }

  auto load_raw = [&](uint32_t stage_off, Raw<BITS, SETS>& r) {
    const uint8_t* gp = smem + stage_off;
    r.a = *reinterpret_cast<const uint4*>(gp + lane * 16);
    if constexpr (BITS == 4) r.b = *reinterpret_cast<const uint4*>(gp + 512 + lane * 16);
    else r.b = *reinterpret_cast<const uint2*>(gp + 512 + lane * 8);
    // scales of rows (g, g+8) sit next to each other: [set][g][2]
#pragma unroll
    for (int sp = 0; sp < SETS; ++sp) r.sc[sp] = *reinterpret_cast<const uint32_t*>(gp + 256 * BITS + 32 * sp + 4 * g);
  };

  // Two granules at once: their bytes become the A fragments of four integer MMAs each (two per
  // group when groups are 64 wide), issued alternately so that neither chain waits for itself;
  // per activation tile, the two sums of each row are joined, scaled by the activation step and
  // the group scale, and the offset term is added.  out[e][b][0 / 1] = rows g / g + 8.
  auto compute_pair = [&](const Raw<BITS, SETS> (&r)[2], const uint32_t (&gi)[2], float (&out)[2][MB][2]) {
    uint32_t R0[2][8], R1[2][8];     // fragment registers of rows g and g + 8
    float2 sc[2][SETS];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      if constexpr (BITS == 4) {
        regs4(r[e].a.x, r[e].a.z, r[e].b.x, r[e].b.z, R0[e]);
        regs4(r[e].a.y, r[e].a.w, r[e].b.y, r[e].b.w, R1[e]);
      } else {
        regs3(r[e].a.x, r[e].a.y, r[e].a.z, R0[e]);
        regs3(r[e].a.w, r[e].b.x, r[e].b.y, R1[e]);
      }
#pragma unroll
      for (int sp = 0; sp < SETS; ++sp) sc[e][sp] = __half22float2(*reinterpret_cast<const __half2*>(&r[e].sc[sp]));
    }
    constexpr int MPS = 4 / SETS;     // MMAs per group
#pragma unroll
    for (int b = 0; b < MB; ++b) {
      uint32_t X[2][8];
      float sx[2], nc[2][2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        {
          // lanes whose B column does not exist read a block of zeros instead (stride 0)
          const uint8_t* xp = smem + xcol_off[b] + gi[e] * xcol_gran[b];
          const uint4 xa = *reinterpret_cast<const uint4*>(xp), xb = *reinterpret_cast<const uint4*>(xp + xcol_plane[b]);
          X[e][0] = xa.x; X[e][1] = xa.y; X[e][2] = xa.z; X[e][3] = xa.w;
          X[e][4] = xb.x; X[e][5] = xb.y; X[e][6] = xb.z; X[e][7] = xb.w;
        }
        const uint8_t* qp = smem + xq_off + (gi[e] * 4 * MB + 4 * b) * 16u;
        if constexpr (SETS == 2) {
          const float4 qv = *reinterpret_cast<const float4*>(qp);
          sx[e] = qv.x; nc[e][0] = qv.y; nc[e][1] = qv.z;
        } else {
          const float2 qv = *reinterpret_cast<const float2*>(qp);
          sx[e] = qv.x; nc[e][0] = qv.y; nc[e][1] = 0.f;
        }
        out[e][b][0] = out[e][b][1] = 0.f;
      }
#pragma unroll
      for (int sp = 0; sp < SETS; ++sp) {
        int acc[2][4];
#pragma unroll
        for (int e = 0; e < 2; ++e)
          imma16832(acc[e], R0[e][2 * MPS * sp], R1[e][2 * MPS * sp], R0[e][2 * MPS * sp + 1], R1[e][2 * MPS * sp + 1],
                    X[e][2 * MPS * sp], X[e][2 * MPS * sp + 1], 0, 0, 0, 0);
#pragma unroll
        for (int m = MPS * sp + 1; m < MPS * (sp + 1); ++m)
#pragma unroll
          for (int e = 0; e < 2; ++e)
            imma16832(acc[e], R0[e][2 * m], R1[e][2 * m], R0[e][2 * m + 1], R1[e][2 * m + 1], X[e][2 * m], X[e][2 * m + 1],
                      acc[e][0], acc[e][1], acc[e][2], acc[e][3]);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float v0 = fmaf((float)(acc[e][0] * 128 + acc[e][1]), sx[e], nc[e][sp]);
          const float v1 = fmaf((float)(acc[e][2] * 128 + acc[e][3]), sx[e], nc[e][sp]);
          out[e][b][0] = fmaf(sc[e][sp].x, v0, out[e][b][0]);
          out[e][b][1] = fmaf(sc[e][sp].y, v1, out[e][b][1]);
        }
      }
    }
  };

  // ---- piece bookkeeping: every warp closes every piece, in order, whether or not it held one of
  // the piece's granules (partials are parked per warp and summed in warp order)
  int pending = 0;
  bool cher_ready = false;
  auto close_piece = [&](uint32_t i) {
    {
      float* dst = slots + ((size_t)((i % p.nslot) * NCW + warp) * p.M) * 16;
#pragma unroll
      for (int b = 0; b < MB; ++b) {
        const int m = 4 * b + t;
        if (m < p.M) {
          dst[m * 16 + g] = tot[b][0];
          dst[m * 16 + g + 8] = tot[b][1];
        }
        tot[b][0] = tot[b][1] = 0.f;
      }
      if (did_cher) {           // warp-uniform: this warp held the sub-tile's first granule
        __syncwarp();
#pragma unroll
        for (int b = 0; b < MBH; ++b) {
          const int m0 = 8 * b + 2 * t;
          if (m0 < p.M) {
            dst[m0 * 16 + g] += ctot[b][0];
            dst[m0 * 16 + g + 8] += ctot[b][2];
          }
          if (m0 + 1 < p.M) {
            dst[(m0 + 1) * 16 + g] += ctot[b][1];
            dst[(m0 + 1) * 16 + g + 8] += ctot[b][3];
          }
          ctot[b][0] = ctot[b][1] = ctot[b][2] = ctot[b][3] = 0.f;
        }
        did_cher = false;
      }
    }
    ++pending;
    const Piece pc = piece_of(i, j_hi, NG, ga, gb);
    const bool post_now = (i == 0) && (pc.end < pc.sub0 + NG);   // piece 0 ends before its sub-tile does
    if (!(post_now || pending == p.nslot || i == npieces - 1)) return;

    // ---- emit the pending pieces
    if (tid == 0 && i == npieces - 1) stamp(p, 6);
    bar_consumers<NCONS>();
    // one thread per (pending piece, activation row, weight row): all pieces are emitted at once
    const uint32_t first = i + 1 - pending;
    const uint32_t n_out = (uint32_t)pending * (uint32_t)p.M * 16u;
    for (uint32_t e = (uint32_t)tid; e < n_out; e += NCONS) {
      const uint32_t pl = e / ((uint32_t)p.M * 16u), mr = e - pl * (uint32_t)p.M * 16u;
      const uint32_t ii = first + pl;
      const int m = (int)(mr >> 4), r = (int)(mr & 15u);
      const Piece q = piece_of(ii, j_hi, NG, ga, gb);
      float v = 0.f;
      {
        const float* sl = slots + ((size_t)((ii % p.nslot) * NCW) * p.M + m) * 16 + r;
#pragma unroll
        for (int w = 0; w < NCW; ++w) v += sl[(size_t)w * p.M * 16];
      }
      if (q.end < q.sub0 + NG) {
        // an earlier part of a cut sub-tile: hand the partial to the CTA that holds its end
        p.partial[(size_t)cta * 256 + mr] = v;
      } else {
        if (q.start > q.sub0) {
          mbar_wait(bar_base + 16 * S + 8, 0, &s_abort, p.status);
          v += reinterpret_cast<const float*>(smem + p.off_pf)[mr];
        }
        const int n = (int)q.j * 16 + r;
        if (n < p.N) {
          __half* yp = p.y + (size_t)m * p.ldy + n;
          if (p.accumulate) v += __half2float(*yp);
          *yp = __float2half(v);
        }
      }
    }
    // what thread 0 has to publish afterwards: did a pending piece post a partial, and which flags
    // of earlier CTAs the finished head sub-tile consumed
    uint32_t reset_lo = 1, reset_hi = 0;
    bool posted = false;
    if (tid == 0) {
      for (uint32_t ii = first; ii <= i; ++ii) {
        const Piece q = piece_of(ii, j_hi, NG, ga, gb);
        if (q.end < q.sub0 + NG) {
          posted = true;
        } else if (q.start > q.sub0) {
          reset_lo = (uint32_t)((((uint64_t)q.sub0 + 1) * grid - 1) / p.T);
          reset_hi = cta - 1;
        }
      }
    }
    bar_consumers<NCONS>();
    if (tid == 0) {
      if (posted) {
        __threadfence();
        st_release(p.flag + cta, 1u);
      }
      for (uint32_t c = reset_lo; c <= reset_hi && reset_lo <= reset_hi; ++c) p.flag[c] = 0u;
      if (i == npieces - 1) stamp(p, 7);
    }
    pending = 0;
  };

  // ---- this warp's granules.  Ring stage (it mod S) holds positions [it * CH, (it + 1) * CH) of the
  // CTA's sequence, CH = 2 * NCW; warp w owns the pair at 2w of every stage.  Per stage a warp
  // waits for the copy, pulls its two granules into registers, hands the slot back, and only then
  // does the math.  Which granule of which piece a position is comes from the schedule table.
  // The granule that starts a sub-tile also adds the sub-tile's fp16 cherry columns.
  auto add_cherries = [&](uint32_t piece) {
    if (!cher_ready) {
      mbar_wait(bar_base + 16 * S, 0, &s_abort, p.status);
      cher_ready = true;
    }
    did_cher = true;
    const uint8_t* blk = smem + p.off_cher + (size_t)(j_hi - piece - jc_lo) * p.cher_bytes;
    for (int jj = 0; jj < p.Cp / 16; ++jj) {
      const uint4 a = *reinterpret_cast<const uint4*>(blk + jj * 512 + lane * 16);
#pragma unroll
      for (int b = 0; b < MBH; ++b) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(smem + xc_off[b] + 32 * jj);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(smem + xc_off[b] + 32 * jj + 16);
        mma16816(ctot[b], a.x, a.y, a.z, a.w, b0, b1);
      }
    }
  };

  uint32_t nclosed = 0;
  {
    const uint32_t n_iters = (total + CH - 1) / CH;
    const uint32_t sched_off = (uint32_t)p.off_sched + 8u * (uint32_t)warp;
    uint32_t stage = 0, phase = 0;
    uint32_t pa = 2u * (uint32_t)warp;
    for (uint32_t it = 0; it < n_iters; ++it, pa += CH) {
      mbar_wait(bar_base + 8 * stage, phase, &s_abort, p.status);
      if (it == 0 && tid == 0) stamp(p, 5);
      const bool va = pa < total, vb = pa + 1 < total;     // warp-uniform
      Raw<BITS, SETS> r[2];
      const uint32_t soff = ring_off + stage * CH * GB;
      load_raw(va ? soff : ring_off, r[0]);                 // (a stale slot is harmless: its result is dropped)
      load_raw(vb ? soff + GB : ring_off, r[1]);
      const uint2 se = *reinterpret_cast<const uint2*>(smem + sched_off + it * (CH * 4));
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_base + 8 * (S + stage));
      if (++stage == S) { stage = 0; phase ^= 1; }
      if (!va) continue;
      const uint32_t gi[2] = {se.x & 1023u, se.y & 1023u};
      float out[2][MB][2];
      compute_pair(r, gi, out);
      while (nclosed < (se.x >> 10)) close_piece(nclosed++);
#pragma unroll
      for (int b = 0; b < MB; ++b) { tot[b][0] += out[0][b][0]; tot[b][1] += out[0][b][1]; }
      if (gi[0] == 0 && p.Cp > 0) add_cherries(se.x >> 10);
      if (vb) {
        while (nclosed < (se.y >> 10)) close_piece(nclosed++);
#pragma unroll
        for (int b = 0; b < MB; ++b) { tot[b][0] += out[1][b][0]; tot[b][1] += out[1][b][1]; }
        if (gi[1] == 0 && p.Cp > 0) add_cherries(se.y >> 10);
      }
    }
  }
  for (; nclosed < npieces; ++nclosed) close_piece(nclosed);
}

// ------------------------------------------------------------------ host side
struct DeviceInfo {
  int sms = 0;
  int max_smem = 0;
  bool ok = false;
};

DeviceInfo device_info(int dev) {
  static DeviceInfo cache[64];
  if (dev < 0 || dev >= 64) return DeviceInfo();
  if (!cache[dev].ok) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return DeviceInfo();
    cache[dev].sms = prop.multiProcessorCount;
    cache[dev].max_smem = (int)prop.sharedMemPerBlockOptin - 1024;
    cache[dev].ok = true;
  }
  return cache[dev];
}

typedef void (*KernelFn)(const MatvecParams);

// The product shape for launches of up to four activation rows: 19 consumer warps (a pair of granules per
// warp per ring stage) with the whole SM to themselves, 96 registers; it measured fastest on the LLaMA-7B
// layers (more warps hide more of the per-instruction latency of the unpack code than sharing the SM
// with the next launch's prefetch gains).  Launches of more than four activation rows use 11 consumer
// warps and the whole register file.
constexpr int SMALL_NCW = 19, SMALL_REGS = 96, LARGE_NCW = 11;
constexpr int SMEM_TARGET_KB = 220;      // shared memory per CTA (the whole SM)
constexpr int MAX_STAGES = 16;           // ring stages
constexpr int INFLIGHT = 2;              // ring stages outstanding at a time

KernelFn pick_small(int bits, int sets) {
  if (bits == 4) return sets == 1 ? cq_matvec_kernel<4, 1, 1, SMALL_NCW, SMALL_REGS> : cq_matvec_kernel<4, 2, 1, SMALL_NCW, SMALL_REGS>;
  return sets == 1 ? cq_matvec_kernel<3, 1, 1, SMALL_NCW, SMALL_REGS> : cq_matvec_kernel<3, 2, 1, SMALL_NCW, SMALL_REGS>;
}
template <int MB>
KernelFn pick_large(int bits, int sets) {
  if (bits == 4) return sets == 1 ? cq_matvec_kernel<4, 1, MB, LARGE_NCW, 128> : cq_matvec_kernel<4, 2, MB, LARGE_NCW, 128>;
  return sets == 1 ? cq_matvec_kernel<3, 1, MB, LARGE_NCW, 128> : cq_matvec_kernel<3, 2, MB, LARGE_NCW, 128>;
}

// mb = activation tiles of four rows: 1, 2 or 4.  Returns the kernel and its consumer warp count.
KernelFn pick_kernel(int bits, int sets, int mb, int* ncw) {
  if (mb == 1) {
    *ncw = SMALL_NCW;
    return pick_small(bits, sets);
  }
  *ncw = LARGE_NCW;
  return mb == 2 ? pick_large<2>(bits, sets) : pick_large<4>(bits, sets);
}

int align_up(int v, int a) { return (v + a - 1) / a * a; }

int tiles_of(int M) { return M <= 4 ? 1 : (M <= 8 ? 2 : 4); }

// Shared-memory plan for M activation rows with `nslot` parking slots for finished pieces;
// returns total bytes or -1 if it cannot fit.
int plan_smem_slots(const cq_layer* L, int M, int grid, int max_smem, int ncw, int target_kb, int max_stages,
                    int nslot, MatvecParams* p) {
  const uint32_t T = (uint32_t)L->n_sub * (uint32_t)L->n_gran;
  const uint32_t per = (T + grid - 1) / grid;
  const int max_pieces = (int)((per + L->n_gran - 1) / L->n_gran) + 1;
  const int mb = tiles_of(M);
  p->nslot = max_pieces < nslot ? max_pieces : nslot;
  p->max_cher = max_pieces;
  p->xb_gran = 256 * M;
  p->xc_stride = L->Cp + 8;
  const int chunk = 2 * ncw * L->gran_bytes;
  int off = 0;
  p->off_cher = off; off = align_up(off + p->max_cher * L->cher_bytes, 128);
  p->off_zero = off; off = align_up(off + 16, 128);
  p->off_sched = off; off = align_up(off + ((int)per + 2 * ncw) * 4, 128);
  p->off_xb = off;   off = align_up(off + L->n_gran * p->xb_gran, 128);
  p->off_xq = off;   off = align_up(off + L->n_gran * 4 * mb * 16, 128);
  p->off_xc = off;   off = align_up(off + M * p->xc_stride * 2, 128);
  p->off_slot = off; off = align_up(off + p->nslot * ncw * M * 64, 128);
  p->off_pf = off;   off = align_up(off + 256 * 4, 128);
  p->off_bar = off;  off = align_up(off + (2 * 16 + 2) * 8, 128);
  p->off_ring = off;
  const int fixed = off;
  // Ring: target_kb per CTA (the default takes the whole SM; <= 111 lets two launches share an
  // SM, which only pays while the ring still holds enough bytes in flight to cover HBM latency).
  int budget = target_kb * 1024;
  if (budget > max_smem) budget = max_smem;
  if (budget - fixed < 48 * 1024) budget = max_smem;
  int stages = (budget - fixed) / chunk;
  if (stages > 16) stages = 16;
  if (stages > max_stages) stages = max_stages;
  const uint32_t max_chunks = per / (2 * ncw) + 2;
  if ((uint32_t)stages > max_chunks) stages = (int)max_chunks;
  // One stage is being refilled while another is read: at least two stages are required.
  if (stages < 2) stages = 2;
  if (fixed + stages * chunk > max_smem) return -1;
  p->stages = stages;
  return fixed + stages * chunk;
}

// Fewer parking slots (more, smaller output rounds) when many activation rows make them large.
int plan_smem(const cq_layer* L, int M, int grid, int max_smem, int ncw, int target_kb, int max_stages,
              MatvecParams* p) {
  for (int nslot = 8; nslot >= 1; nslot >>= 1) {
    const int smem = plan_smem_slots(L, M, grid, max_smem, ncw, target_kb, max_stages, nslot, p);
    if (smem >= 0) return smem;
  }
  return -1;
}

// Opt in to the dynamic shared memory the plan needs, and ask for the largest shared-memory
// carve-out so that a second CTA (the next launch in the stream) fits beside this one.
cudaError_t prepare_kernel(KernelFn fn, int smem) {
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

}  // namespace

#ifdef CQ_MATVEC_TRACE
// Instrumented builds only (not part of the library's interface): when a device buffer of 1024 x 64
// uint64 is set, every CTA of the following matvec launches stores %globaltimer stamps of its phases
// there: 0 entry, 1 barriers ready, 2 layer constants staged, 3 previous kernel done, 4 activations
// staged, 5 first weights landed, 6 last granule done, 7 exit, 8/9 first and last bulk copy issued,
// 16+c consumer passed the wait for ring copy c, 40+c copy c issued (c < 24).  Not thread-safe.
extern "C" int cq_trace_set_timeline(void* device_buffer) {
  cq_g_timeline = (unsigned long long*)device_buffer;
  return CQ_OK;
}
#endif

extern "C" size_t cq_scratch_bytes(void) {
  // stream kernel: up to 1024 CTAs x 256 floats of partial, flags behind them at 1 MiB;
  // tile kernel: up to 256 CTAs x 2048 floats, flags behind them at 2 MiB
  return (size_t)256 * 2048 * sizeof(float) + 1024 * sizeof(uint32_t);
}

// Launches over at most 16 activation rows (fewer when the shared-memory plan needs it);
// the caller (cq_layer_matvec) walks larger batches.
static int launch_rows(const cq_layer* L, const __half* x, int ldx, __half* y, int ldy, int M,
                       int accumulate, void* scratch, uint32_t* status, cudaStream_t st,
                       int* rows_done) {
  int dev = 0;
  CQ_CUDA_TRY(cudaGetDevice(&dev));
  const DeviceInfo di = device_info(dev);
  if (!di.ok) return CQ_ERR_NO_DEVICE;
  const uint32_t T = (uint32_t)L->n_sub * (uint32_t)L->n_gran;
  int grid = di.sms < 1024 ? di.sms : 1024;
  if ((uint32_t)grid > T) grid = (int)T;

  MatvecParams p;
  int rows = M < 16 ? M : 16;
  int smem = -1, ncw = 0;
  KernelFn fn = nullptr;
  for (; rows >= 1; --rows) {
    fn = pick_kernel(L->bits, L->sets, tiles_of(rows), &ncw);
    smem = plan_smem(L, rows, grid, di.max_smem, ncw, SMEM_TARGET_KB, MAX_STAGES, &p);
    if (smem >= 0) break;
  }
  if (smem < 0) return CQ_ERR_TOO_LARGE;
  const uint8_t* blob = (const uint8_t*)L->blob;
  p.stream = blob + L->off_stream;
  p.cstream = blob + L->off_cherry;
  p.cidx = (const uint16_t*)(blob + L->off_cidx);
  p.osh = (const uint32_t*)(blob + L->off_osh);
  p.x = x; p.y = y;
  p.partial = (float*)scratch;
  p.flag = (uint32_t*)((uint8_t*)scratch + (size_t)1024 * 256 * sizeof(float));
  p.status = status;
#ifdef CQ_MATVEC_TRACE
  p.timeline = cq_g_timeline;
#else
  p.timeline = nullptr;
#endif
  p.M = rows; p.K = L->K; p.N = L->N; p.C = L->C; p.Cp = L->Cp; p.Kp = L->Kp;
  p.n_gran = L->n_gran; p.n_sub = L->n_sub; p.gran_bytes = L->gran_bytes; p.cher_bytes = L->cher_bytes;
  p.ldx = ldx; p.ldy = ldy; p.accumulate = accumulate;
  p.T = T;
  p.inflight = INFLIGHT;

  CQ_CUDA_TRY(prepare_kernel(fn, smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3((ncw + 1) * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, fn, p));
  *rows_done = rows;
  return CQ_OK;
}

extern "C" int cq_layer_matvec(const cq_layer* L, const void* x, int ldx, void* y, int ldy, int M,
                               int accumulate, void* scratch, uint32_t* status_word,
                               cq_stream_t stream) {
  if (!L || !L->blob || !x || !y || !scratch) return CQ_ERR_BAD_ARG;
  if (M < 1 || ldx < L->K || ldy < L->N) return CQ_ERR_BAD_ARG;
  if (((uintptr_t)x & 1) || ((uintptr_t)y & 1)) return CQ_ERR_BAD_ARG;
  const __half* xp = (const __half*)x;
  __half* yp = (__half*)y;
  int done = 0;
  while (done < M) {
    int rows = 0;
    const int rc = launch_rows(L, xp + (size_t)done * ldx, ldx, yp + (size_t)done * ldy, ldy,
                               M - done, accumulate, scratch, status_word, (cudaStream_t)stream, &rows);
    if (rc != CQ_OK) return rc;
    done += rows;
  }
  return CQ_OK;
}

// Self-test of the bounded waits: one warp waits on a barrier that nothing ever completes.  The
// wait gives up after about a second, sets bit 0 of the status word and the kernel returns normally,
// which is what every wait of the matvec kernels does when its partner never shows up.
namespace {
__global__ void bounded_wait_selftest_kernel(uint32_t* status) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  mbar_wait(b, 0, &abort_flag, status);
}
}  // namespace

extern "C" int cq_selftest_bounded_wait(uint32_t* status_word, cq_stream_t stream) {
  if (!status_word) return CQ_ERR_BAD_ARG;
  bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status_word);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}

// ---------------------------------------------------------------------------------------------
// Variant of cq_layer_matvec for callers that own no device scratch and may not obtain any.
//
// Who that is: a host runtime that plans all of its device memory up front and forbids
// allocation once serving has begun (an inference server with a fixed arena, a plugin loaded
// into somebody else's process that must not disturb that process's memory pool), and code that
// runs where an allocation would synchronise the device or fail outright, such as a latency-
// critical decode loop.  cq_layer_matvec asks such a caller for cq_scratch_bytes() of zeroed
// memory; this entry point brings its own instead: the array below lives in the library's
// device image, so it exists on every device as soon as the module is loaded there, and no
// allocating call (runtime, driver or framework) is made here, ever.
//
// Limits (beyond them the call returns CQ_ERR_STATIC_LIMIT and launches nothing):
//   * at most CQ_STATIC_MAX_ROWS (16) activation rows per call: one kernel launch;
//   * at most CQ_STATIC_MAX_CTAS (256) CTAs, i.e. a device with at most 256 SMs.
// Layout of the array: [256 CTAs][256 floats] partial sums | 256 flags | (pad to 256 B).
//
// Sharing: every call on a device uses the same array.  Partial sums are written before they are
// read, the flags must be zero when the kernel starts: each call clears them on the stream ahead of
// its launch, so a call that follows one that ended in a device time-out still starts clean.  Two
// calls that can run at the same time on one device (different streams, different host threads)
// race on the array and give wrong sums: serialise them.
//
// Set-up: the first call on each device resolves the array's device address
// (cudaGetSymbolAddress, with that device current).  That first call should be made before any
// stream capture is begun on the device.
static constexpr int CQ_STATIC_MAX_ROWS = 16;
static constexpr int CQ_STATIC_MAX_CTAS = 256;
static constexpr size_t CQ_STATIC_PARTIAL_BYTES = (size_t)CQ_STATIC_MAX_CTAS * 256 * sizeof(float);
static constexpr size_t CQ_STATIC_FLAG_BYTES = (size_t)CQ_STATIC_MAX_CTAS * sizeof(uint32_t);
static constexpr size_t CQ_STATIC_BYTES = CQ_STATIC_PARTIAL_BYTES + CQ_STATIC_FLAG_BYTES;  // 263,168 B

static __device__ __align__(256) unsigned char cq_static_scratch[CQ_STATIC_BYTES];

namespace {
constexpr int CQ_STATIC_MAX_DEVICES = 64;
std::mutex g_static_mu;
unsigned char* g_static_ptr[CQ_STATIC_MAX_DEVICES] = {};

// Device address of cq_static_scratch on the current device (resolved once per device).
int static_scratch_ptr(int dev, unsigned char** out) {
  if (dev < 0 || dev >= CQ_STATIC_MAX_DEVICES) return CQ_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[dev]) {
    unsigned char* ptr = nullptr;
    CQ_CUDA_TRY(cudaGetSymbolAddress((void**)&ptr, cq_static_scratch));
    if (!ptr || ((uintptr_t)ptr & 255)) return CQ_ERR_CUDA;
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return CQ_OK;
}
}  // namespace

extern "C" int cq_layer_matvec_static(const cq_layer* L, const void* x, int ldx, void* y, int ldy,
                                      int M, int accumulate, uint32_t* status_word,
                                      cq_stream_t stream) {
  if (!L || !L->blob || !x || !y) return CQ_ERR_BAD_ARG;
  if (M < 1 || ldx < L->K || ldy < L->N) return CQ_ERR_BAD_ARG;
  if (((uintptr_t)x & 1) || ((uintptr_t)y & 1)) return CQ_ERR_BAD_ARG;
  if (M > CQ_STATIC_MAX_ROWS) return CQ_ERR_STATIC_LIMIT;
  int dev = 0;
  CQ_CUDA_TRY(cudaGetDevice(&dev));
  const DeviceInfo di = device_info(dev);
  if (!di.ok) return CQ_ERR_NO_DEVICE;
  if (di.sms > CQ_STATIC_MAX_CTAS) return CQ_ERR_STATIC_LIMIT;
  const uint32_t T = (uint32_t)L->n_sub * (uint32_t)L->n_gran;
  int grid = di.sms;
  if ((uint32_t)grid > T) grid = (int)T;

  // one launch must take all M rows: the array has room for one launch's partial sums only
  MatvecParams p;
  int ncw = 0;
  KernelFn fn = pick_kernel(L->bits, L->sets, tiles_of(M), &ncw);
  const int smem = plan_smem(L, M, grid, di.max_smem, ncw, SMEM_TARGET_KB, MAX_STAGES, &p);
  if (smem < 0) return CQ_ERR_STATIC_LIMIT;

  unsigned char* base = nullptr;
  const int rc = static_scratch_ptr(dev, &base);
  if (rc != CQ_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  CQ_CUDA_TRY(cudaMemsetAsync(base + CQ_STATIC_PARTIAL_BYTES, 0, CQ_STATIC_FLAG_BYTES, st));

  const uint8_t* blob = (const uint8_t*)L->blob;
  p.stream = blob + L->off_stream;
  p.cstream = blob + L->off_cherry;
  p.cidx = (const uint16_t*)(blob + L->off_cidx);
  p.osh = (const uint32_t*)(blob + L->off_osh);
  p.x = (const __half*)x; p.y = (__half*)y;
  p.partial = (float*)base;
  p.flag = (uint32_t*)(base + CQ_STATIC_PARTIAL_BYTES);
  p.status = status_word;
  p.timeline = nullptr;
  p.M = M; p.K = L->K; p.N = L->N; p.C = L->C; p.Cp = L->Cp; p.Kp = L->Kp;
  p.n_gran = L->n_gran; p.n_sub = L->n_sub; p.gran_bytes = L->gran_bytes; p.cher_bytes = L->cher_bytes;
  p.ldx = ldx; p.ldy = ldy; p.accumulate = accumulate;
  p.T = T;
  p.inflight = INFLIGHT;

  CQ_CUDA_TRY(prepare_kernel(fn, smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3((ncw + 1) * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  CQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, fn, p));
  return CQ_OK;
}
