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
//    async copies (cp.async.bulk + mbarrier transaction counts), NCW * GPW
//    granules per copy.  It starts before the kernel waits for the previous kernel
//    in the stream (programmatic dependent launch): weights never depend on it.
//  * NCW consumer warps take the granules of a copy round-robin, GPW each.  A lane
//    reads its 16 (4-bit) or 24 (3-bit) bytes, turns codes into fp16 pairs with one
//    AND-OR per pair (exponent trick, offsets folded into a per-group correction
//    computed while the activations are staged), and feeds mma.sync.m16n8k16 with
//    the activations (staged once in shared memory in compact order) as the B
//    operand.  Group scales are applied per granule in fp32.
//  * A range is walked from its last sub-tile to its first.  A sub-tile cut by a
//    range boundary is finished by the CTA that holds its end: CTAs holding an
//    earlier part post their fp32 partial to global scratch early in their walk,
//    the finishing CTA adds the partials in a fixed order late in its walk.  All
//    sums are therefore deterministic.  Every wait is bounded; running out sets
//    a bit in the status word instead of hanging.
#include <cstdlib>
#include <mutex>

#include "cq_common.cuh"

unsigned long long* cq_g_timeline = nullptr;   // tracing buffer, see cq_trace_set_timeline

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
  int stages, nslot, max_cher;
  // shared-memory offsets
  int off_ring, off_cher, off_xs, off_xc, off_cidx, off_osh, off_corr, off_slot, off_pf, off_bar;
  int xs_stride;       // halves per activation row in smem (Kp + 8)
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
  const uint32_t limit = *abort_flag ? 1u : WAIT_LIMIT;
  for (uint32_t it = 0; it < limit; ++it)
    if (mbar_try_wait(bar, parity)) return true;
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
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ void stamp(const MatvecParams& p, int slot) {
  if (p.timeline) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.timeline[(size_t)blockIdx.x * 64 + slot] = t;
  }
}

// ------------------------------------------------------------------ decode
// Codes become fp16 values with one AND-OR each: OR-ing a code field that sits at
// mantissa bit p into the bit pattern of 1024.0 gives the fp16 number 1024 + 2^p * u.
// No subtraction follows.  Instead the activation that meets this code in the MMA is
// pre-multiplied by 2^(c-p) when it is staged, so that the product is
// 2^c * (B + u) * x with B = 2^(10-p), and the excess (B + off) * x, summed per
// group while staging ("corr"), is removed in fp32 when the group scale is applied:
//     y += s * (acc * 2^-c - corr).
// p is a function of the code's position only, so both sides agree by layout.
constexpr uint32_t MAGIC = 0x64006400u;  // (1024, 1024)

template <int BITS> struct Fold;
template <> struct Fold<4> {
  static constexpr int C_EXP = 2;                 // products carry 2^2
  static constexpr float OFF = 7.5f;
};
template <> struct Fold<3> {
  static constexpr int C_EXP = 1;
  static constexpr float OFF = 3.5f;
};
// Mantissa bit p of the code field of pair q.  4-bit: q = (position >> 1) in the lane's
// 16 codes of a 64-column half (even -> 2, odd -> 6).  3-bit: q = 0..15 over the row's 32
// codes of the granule (word slot q % 5 -> 1, 4, 7, 4, 7; pair 15 -> 7).
template <int BITS>
__device__ __forceinline__ int fold_p(int q) {
  if (BITS == 4) return (q & 1) ? 6 : 2;
  const int r = q % 5;
  return q == 15 ? 7 : (r == 0 ? 1 : ((r & 1) ? 4 : 7));
}

// One 4-bit stream word -> 4 fp16 pairs (codes (0,1), (2,3), (4,5), (6,7)): 1024 + 4u, 1024 + 64u, ...
__device__ __forceinline__ void decode4(uint32_t w, uint32_t* out) {
  const uint32_t v1 = w << 2, v2 = w >> 6;
  out[0] = (v1 & 0x003C003Cu) | MAGIC;
  out[1] = (v1 & 0x03C003C0u) | MAGIC;
  out[2] = (v2 & 0x003C003Cu) | MAGIC;
  out[3] = (v2 & 0x03C003C0u) | MAGIC;
}

// Three 3-bit stream words of one row -> 16 fp16 pairs (codes (2q, 2q+1)).
__device__ __forceinline__ void decode3(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t* out) {
  const uint32_t w[3] = {w0, w1, w2};
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const uint32_t v = w[i] >> 6;
    out[5 * i + 0] = (w[i] & 0x000E000Eu) | MAGIC;   // field at bit 1
    out[5 * i + 1] = (w[i] & 0x00700070u) | MAGIC;   // field at bit 4
    out[5 * i + 2] = (w[i] & 0x03800380u) | MAGIC;   // field at bit 7
    out[5 * i + 3] = (v & 0x00700070u) | MAGIC;      // field at bit 10 -> 4
    out[5 * i + 4] = (v & 0x03800380u) | MAGIC;      // field at bit 13 -> 7
  }
  uint32_t r = ((w0 << 7) & 0x00800080u) | MAGIC;    // pair 15: one bit from each word, at bits 7..9
  r |= (w1 << 8) & 0x01000100u;
  r |= (w2 << 9) & 0x02000200u;
  out[15] = r;
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
template <int BITS> struct Raw;
template <> struct Raw<4> { uint4 a, b; uint32_t sc[2]; };
template <> struct Raw<3> { uint2 a, b, c; uint32_t sc[2]; };

template <int BITS, int SETS, int MB, int NCW, int MINB>
__global__ void __launch_bounds__((NCW + 1) * 32, MINB) cq_matvec_kernel(const MatvecParams p) {
  constexpr int NCONS = NCW * 32;
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
    if (p.timeline) p.timeline[(size_t)blockIdx.x * 64 + 10] = (unsigned long long)clock64();
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
  // (g mod S) holds positions [g * NCW, (g + 1) * NCW): position q sits at slot q mod NCW of it
  // and belongs to consumer warp q mod NCW.  A stage is filled by one bulk copy per piece it
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
      for (uint32_t q0 = 0; q0 < total; q0 += NCW) {
        const uint32_t len = min((uint32_t)NCW, total - q0);
        if (!first_pass) mbar_wait(bar_base + 8 * (S + stage), phase, &s_abort, p.status);
        mbar_expect_tx(bar_base + 8 * stage, len * GB);
        uint32_t dst = ring + stage * NCW * GB, left = len;
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
  // Layer constants first (they do not depend on the previous kernel): the sorted cherry
  // columns and, per octet of compact columns, how far its first and last column are shifted
  // in the original row (see cq_common.cuh).
  __half* xs = reinterpret_cast<__half*>(smem + p.off_xs);
  __half* xc = reinterpret_cast<__half*>(smem + p.off_xc);
  float* corr = reinterpret_cast<float*>(smem + p.off_corr);
  uint16_t* cidx_s = reinterpret_cast<uint16_t*>(smem + p.off_cidx);
  uint32_t* osh = reinterpret_cast<uint32_t*>(smem + p.off_osh);
  const int noct = p.Kp >> 3;
  for (int c = tid; c < p.Cp; c += NCONS) cidx_s[c] = p.cidx[c];
  // corr entries of activation rows that do not exist must read as zero
  for (int i = tid; i < (int)NG * SETS * 8 * MB; i += NCONS) corr[i] = 0.f;
  for (int o = tid; o < noct; o += NCONS) osh[o] = p.osh[o];
  bar_consumers<NCONS>();
  if (tid == 0) stamp(p, 2);

  // Everything below may read what the previous kernel in the stream wrote.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (tid == 0) stamp(p, 3);

  // Activations of the cherry columns: issue the loads now, store them after the main gather,
  // so that both cost one trip to L2 together.
  constexpr int XCU = 2;
  __half xcv[XCU];
#pragma unroll
  for (int u = 0; u < XCU; ++u) {
    const int idx = tid + u * NCONS;
    xcv[u] = __float2half(0.f);
    if (idx < p.M * p.Cp) {
      const int m = idx / p.Cp, c = idx - m * p.Cp;
      const uint32_t o = cidx_s[c];
      if (o != CQ_PAD_COL) xcv[u] = __ldg(p.x + (size_t)m * p.ldx + o);
    }
  }
  {
    // xs[m][k'] = 2^(c-p(k')) * x[m][orig(k')] for the compact columns, 8 at a time (zero past K'),
    // and corr[granule][set][m] = sum over the group of (B + off) * x.
    const int nitem = noct * p.M;
    constexpr int U = 4;
    constexpr int CE = Fold<BITS>::C_EXP;
    for (int base = 0; base < nitem; base += NCONS * U) {
      uint32_t v[U][4];
      int dsto[U], mrow[U], oct[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int it = base + u * NCONS + tid;
        dsto[u] = -1;
        mrow[u] = 0;
        oct[u] = 0;
        v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0u;
        if (it < nitem) {
          const int m = (p.M == 1) ? 0 : it / noct;
          const int o = it - m * noct;
          const int k0 = 8 * o;
          dsto[u] = m * p.xs_stride + k0;
          mrow[u] = m;
          oct[u] = o;
          const uint32_t sh = osh[o];
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
              unsigned short h[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                int lo = lo0, hi = lo7;
                while (lo < hi) {
                  const int mid = (lo + hi) >> 1;
                  if ((int)cidx_s[mid] - mid <= k0 + i) lo = mid + 1; else hi = mid;
                }
                h[i] = __ldg(reinterpret_cast<const unsigned short*>(xr + k0 + i + lo));
              }
#pragma unroll
              for (int i = 0; i < 4; ++i) v[u][i] = (uint32_t)h[2 * i] | ((uint32_t)h[2 * i + 1] << 16);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        // first pair index of this octet among the row's pairs of the granule
        const int oo = oct[u] & 15;
        const int q0 = (BITS == 4) ? 0 : 8 * (oo >> 3) + 4 * (oo & 1);
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int pp = fold_p<BITS>(q0 + i);
          const uint32_t sc16 = (uint32_t)((15 + CE - pp) << 10);                 // fp16 2^(c-p)
          const uint32_t scaled = hmul2_u32(v[u][i], sc16 | (sc16 << 16));
          const float coef = __int_as_float((127 + pp - CE) << 23) *              // 2^(p-c) * (B + off)
                             ((float)(1 << (10 - pp)) + Fold<BITS>::OFF);
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&scaled));
          part += (f.x + f.y) * coef;
          v[u][i] = scaled;
        }
        // 16 (8 for 64-wide groups) neighbouring lanes hold the octets of one group of one row
#pragma unroll
        for (int d = 1; d < 16 / SETS; d <<= 1) part += __shfl_xor_sync(0xffffffffu, part, d);
        if (dsto[u] >= 0) {
          *reinterpret_cast<uint4*>(xs + dsto[u]) = make_uint4(v[u][0], v[u][1], v[u][2], v[u][3]);
          if ((oct[u] & (16 / SETS - 1)) == 0) {
            const int gi = oct[u] >> 4, sp = (SETS == 2) ? ((oct[u] >> 3) & 1) : 0;
            corr[(gi * SETS + sp) * 8 * MB + mrow[u]] = part;
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
    const uint32_t o = cidx_s[c];
    xc[m * p.xc_stride + c] = (o != CQ_PAD_COL) ? p.x[(size_t)m * p.ldx + o] : __float2half(0.f);
  }
  bar_consumers<NCONS>();
  if (tid == 0) stamp(p, 4);

  const int g = lane >> 2, t = lane & 3;
  float* slots = reinterpret_cast<float*>(smem + p.off_slot);   // [slot][warp][m][16 rows]

  float tot[MB][4];
#pragma unroll
  for (int b = 0; b < MB; ++b)
#pragma unroll
    for (int r = 0; r < 4; ++r) tot[b][r] = 0.f;

  // Shared-memory byte offsets (relative to `smem`) this lane reads in every granule.
  // B-operand column g of activation tile b is activation row 8b + g; columns past the last
  // row are never read back from the accumulators, so they may carry any existing row.
  uint32_t x_off[MB], xc_off[MB];
#pragma unroll
  for (int b = 0; b < MB; ++b) {
    const int m = (8 * b + g) % p.M;
    x_off[b] = (uint32_t)p.off_xs + (uint32_t)(m * p.xs_stride + 16 * t) * 2u;
    xc_off[b] = (uint32_t)p.off_xc + (uint32_t)(m * p.xc_stride + 2 * t) * 2u;
  }
  const uint32_t corr_off = (uint32_t)p.off_corr + (uint32_t)(2 * t) * 4u;
  const uint32_t lane_w = (BITS == 4) ? (uint32_t)lane * 16u : (uint32_t)lane * 24u;
  const uint32_t ring_off = (uint32_t)p.off_ring + (uint32_t)warp * GB;       // this warp's slot in stage 0

  auto load_raw = [&](uint32_t stage_off, Raw<BITS>& r) {
    const uint8_t* gp = smem + stage_off + lane_w;
    if constexpr (BITS == 4) {
      r.a = *reinterpret_cast<const uint4*>(gp);
      r.b = *reinterpret_cast<const uint4*>(gp + 512);
    } else {
      r.a = *reinterpret_cast<const uint2*>(gp);
      r.b = *reinterpret_cast<const uint2*>(gp + 8);
      r.c = *reinterpret_cast<const uint2*>(gp + 16);
    }
    // scales of rows (g, g+8) sit next to each other: [set][g][2]
    const uint8_t* sp = smem + stage_off + 256 * BITS + 4 * g;
    r.sc[0] = *reinterpret_cast<const uint32_t*>(sp);
    r.sc[1] = (SETS == 2) ? *reinterpret_cast<const uint32_t*>(sp + 32) : r.sc[0];
  };

  // One granule: 8 MMAs (two accumulators per 64-column half, so that no MMA waits for the one
  // issued just before it), then the group scales and the correction.
  auto compute = [&](const Raw<BITS>& r, uint32_t gi) {
    uint32_t A0[16], A1[16];   // fp16 pairs of rows g and g+8 (8 per 64-column half)
    if constexpr (BITS == 4) {
      decode4(r.a.x, A0);      decode4(r.a.y, A0 + 4);  decode4(r.a.z, A1);      decode4(r.a.w, A1 + 4);
      decode4(r.b.x, A0 + 8);  decode4(r.b.y, A0 + 12); decode4(r.b.z, A1 + 8);  decode4(r.b.w, A1 + 12);
    } else {
      decode3(r.a.x, r.a.y, r.b.x, A0);
      decode3(r.b.y, r.c.x, r.c.y, A1);
    }
    float acc[2][2][MB][4];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int b = 0; b < MB; ++b)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[h][j][b][e] = 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t X[MB][8];
#pragma unroll
      for (int b = 0; b < MB; ++b) {
        const uint8_t* xp = smem + x_off[b] + gi * 256u + h * 128;
        const uint4 xa = *reinterpret_cast<const uint4*>(xp), xb = *reinterpret_cast<const uint4*>(xp + 16);
        X[b][0] = xa.x; X[b][1] = xa.y; X[b][2] = xa.z; X[b][3] = xa.w;
        X[b][4] = xb.x; X[b][5] = xb.y; X[b][6] = xb.z; X[b][7] = xb.w;
      }
#pragma unroll
      for (int m = 0; m < 4; ++m)
#pragma unroll
        for (int b = 0; b < MB; ++b)
          mma16816(acc[h][m & 1][b], A0[8 * h + 2 * m], A1[8 * h + 2 * m], A0[8 * h + 2 * m + 1], A1[8 * h + 2 * m + 1],
                   X[b][2 * m], X[b][2 * m + 1]);
    }
    const float inv = 1.f / (float)(1 << Fold<BITS>::C_EXP);
    const float2 s_lo = __half22float2(*reinterpret_cast<const __half2*>(&r.sc[0]));
    const float2 s_hi = __half22float2(*reinterpret_cast<const __half2*>(&r.sc[1]));
#pragma unroll
    for (int b = 0; b < MB; ++b) {
      // corr: [granule][set][8 * MB] floats; this lane's columns are 8b + 2t, + 1
      const uint8_t* cp = smem + corr_off + (gi * SETS * 8 * MB + 8 * b) * 4u;
      const float2 c_lo = *reinterpret_cast<const float2*>(cp);
      float a0[4], a1[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        a0[e] = acc[0][0][b][e] + acc[0][1][b][e];
        a1[e] = acc[1][0][b][e] + acc[1][1][b][e];
      }
      if (SETS == 2) {
        const float2 c_hi = *reinterpret_cast<const float2*>(cp + 8 * MB * 4);
        tot[b][0] += s_lo.x * (a0[0] * inv - c_lo.x) + s_hi.x * (a1[0] * inv - c_hi.x);
        tot[b][1] += s_lo.x * (a0[1] * inv - c_lo.y) + s_hi.x * (a1[1] * inv - c_hi.y);
        tot[b][2] += s_lo.y * (a0[2] * inv - c_lo.x) + s_hi.y * (a1[2] * inv - c_hi.x);
        tot[b][3] += s_lo.y * (a0[3] * inv - c_lo.y) + s_hi.y * (a1[3] * inv - c_hi.y);
      } else {
        tot[b][0] += s_lo.x * ((a0[0] + a1[0]) * inv - c_lo.x);
        tot[b][1] += s_lo.x * ((a0[1] + a1[1]) * inv - c_lo.y);
        tot[b][2] += s_lo.y * ((a0[2] + a1[2]) * inv - c_lo.x);
        tot[b][3] += s_lo.y * ((a0[3] + a1[3]) * inv - c_lo.y);
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
        const int m0 = 8 * b + 2 * t;
        if (m0 < p.M) {
          dst[m0 * 16 + g] = tot[b][0];
          dst[m0 * 16 + g + 8] = tot[b][2];
        }
        if (m0 + 1 < p.M) {
          dst[(m0 + 1) * 16 + g] = tot[b][1];
          dst[(m0 + 1) * 16 + g + 8] = tot[b][3];
        }
        tot[b][0] = tot[b][1] = tot[b][2] = tot[b][3] = 0.f;
      }
    }
    ++pending;
    const Piece pc = piece_of(i, j_hi, NG, ga, gb);
    const bool post_now = (i == 0) && (pc.end < pc.sub0 + NG);   // piece 0 ends before its sub-tile does
    if (!(post_now || pending == p.nslot || i == npieces - 1)) return;

    // ---- emit the pending pieces
    if (tid == 0 && i == npieces - 1) stamp(p, 6);
    bar_consumers<NCONS>();
    uint32_t reset_lo = 1, reset_hi = 0;    // flags to clear afterwards (finishing CTA only)
    bool posted = false;
    if (tid < 256) {
      for (uint32_t ii = i + 1 - pending; ii <= i; ++ii) {
        const Piece q = piece_of(ii, j_hi, NG, ga, gb);
        const int m = tid >> 4, r = tid & 15;
        float v = 0.f;
        if (m < p.M) {
          const float* sl = slots + ((size_t)((ii % p.nslot) * NCW) * p.M + m) * 16 + r;
#pragma unroll
          for (int w = 0; w < NCW; ++w) v += sl[(size_t)w * p.M * 16];
        }
        if (q.end < q.sub0 + NG) {
          // an earlier part of a cut sub-tile: hand the partial to the CTA that holds its end
          p.partial[(size_t)cta * 256 + tid] = v;
          posted = true;
        } else {
          if (q.start > q.sub0) {
            const uint32_t c_first = (uint32_t)((((uint64_t)q.sub0 + 1) * grid - 1) / p.T);
            reset_lo = c_first;
            reset_hi = cta - 1;
            mbar_wait(bar_base + 16 * S + 8, 0, &s_abort, p.status);
            v += reinterpret_cast<const float*>(smem + p.off_pf)[tid];
          }
          const int n = (int)q.j * 16 + r;
          if (m < p.M && n < p.N) {
            __half* yp = p.y + (size_t)m * p.ldy + n;
            if (p.accumulate) v += __half2float(*yp);
            *yp = __float2half(v);
          }
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
      if (i == npieces - 1) {
        stamp(p, 7);
        if (p.timeline) p.timeline[(size_t)blockIdx.x * 64 + 11] = (unsigned long long)clock64();
      }
    }
    pending = 0;
  };

  // ---- this warp's granules: positions warp, warp + NCW, ... of the CTA's sequence.  While
  // granule i is computed, the words of granule i+1 are already on their way from shared memory
  // (its ring slot is released as soon as they are requested) and the barrier of granule i+2's
  // stage is being probed; the probe's answer is only looked at after the math.
  uint32_t pi = 0;                         // piece of the current position
  Piece pc = piece_of(0, j_hi, NG, ga, gb);
  uint32_t pstart = 0;                     // sequence position where piece pi starts
  if ((uint32_t)warp < total) {
    uint32_t pos = (uint32_t)warp, stage = 0, phase = 0;
    Raw<BITS> cur, nxt;
    mbar_wait(bar_base, 0, &s_abort, p.status);
    if (tid == 0) stamp(p, 5);
    load_raw(ring_off, cur);
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_base + 8 * S);
    if (pos + NCW < total) mbar_wait(bar_base + 8 * (1 % S), (1 / S) & 1, &s_abort, p.status);
    for (;;) {
      while (pos >= pstart + (pc.end - pc.start)) {
        close_piece(pi);
        pstart += pc.end - pc.start;
        pc = piece_of(++pi, j_hi, NG, ga, gb);
      }
      const uint32_t gi = pc.start - pc.sub0 + (pos - pstart);     // granule inside the sub-tile
      const bool has_next = pos + NCW < total, has_next2 = pos + 2 * NCW < total;
      uint32_t nstage = stage + 1, nphase = phase;
      if (nstage == S) { nstage = 0; nphase ^= 1; }
      uint32_t n2stage = nstage + 1, n2phase = nphase;
      if (n2stage == S) { n2stage = 0; n2phase ^= 1; }
      if (has_next) {                      // its stage is known to have landed
        load_raw(ring_off + nstage * NCW * GB, nxt);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_base + 8 * (S + nstage));
      }
      bool ready2 = false;
      if (has_next2) ready2 = mbar_try_wait(bar_base + 8 * n2stage, n2phase);
      compute(cur, gi);
      // The granule that starts a sub-tile also adds the sub-tile's fp16 cherry columns.
      if (gi == 0 && p.Cp > 0) {
        if (!cher_ready) {
          mbar_wait(bar_base + 16 * S, 0, &s_abort, p.status);
          cher_ready = true;
        }
        const uint8_t* blk = smem + p.off_cher + (size_t)(pc.j - jc_lo) * p.cher_bytes;
        for (int jj = 0; jj < p.Cp / 16; ++jj) {
          const uint4 a = *reinterpret_cast<const uint4*>(blk + jj * 512 + lane * 16);
#pragma unroll
          for (int b = 0; b < MB; ++b) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(smem + xc_off[b] + 32 * jj);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(smem + xc_off[b] + 32 * jj + 16);
            mma16816(tot[b], a.x, a.y, a.z, a.w, b0, b1);
          }
        }
      }
      if (!has_next) break;
      if (has_next2 && !ready2) mbar_wait_slow(bar_base + 8 * n2stage, n2phase, &s_abort, p.status);
      cur = nxt;
      pos += NCW; stage = nstage; phase = nphase;
    }
  }
  for (; pi < npieces; ++pi) close_piece(pi);
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

// Kernel shapes: consumer warps (one granule per warp per ring stage).
struct Shape { int ncw, gpw; };
constexpr Shape SHAPES[] = {{8, 1}, {12, 1}, {16, 1}};
constexpr int N_SHAPES = sizeof(SHAPES) / sizeof(SHAPES[0]);

template <int NCW, int MINB>
KernelFn pick_bits(int bits, int sets, int mb) {
  if (bits == 4) {
    if (sets == 1) return mb == 1 ? cq_matvec_kernel<4, 1, 1, NCW, MINB> : cq_matvec_kernel<4, 1, 2, NCW, MINB>;
    return mb == 1 ? cq_matvec_kernel<4, 2, 1, NCW, MINB> : cq_matvec_kernel<4, 2, 2, NCW, MINB>;
  }
  if (sets == 1) return mb == 1 ? cq_matvec_kernel<3, 1, 1, NCW, MINB> : cq_matvec_kernel<3, 1, 2, NCW, MINB>;
  return mb == 1 ? cq_matvec_kernel<3, 2, 1, NCW, MINB> : cq_matvec_kernel<3, 2, 2, NCW, MINB>;
}

KernelFn pick_kernel(int shape, int bits, int sets, int mb) {
  switch (shape) {
    case 0: return pick_bits<8, 1>(bits, sets, mb);
    case 1: return pick_bits<12, 1>(bits, sets, mb);
    default: return pick_bits<16, 1>(bits, sets, mb);
  }
}

// Tuning knobs read once from the environment (for experiments; defaults are the product):
//   CQ_SHAPE  index into SHAPES      CQ_SMEM_KB  shared-memory target per CTA
//   CQ_PDL    0 disables programmatic dependent launch
struct Knobs { int shape, smem_kb, pdl, max_stages; };
Knobs knobs() {
  static Knobs k = [] {
    Knobs v{0, 112, 1, 16};
    if (const char* e = getenv("CQ_SHAPE")) v.shape = atoi(e);
    if (const char* e = getenv("CQ_SMEM_KB")) v.smem_kb = atoi(e);
    if (const char* e = getenv("CQ_PDL")) v.pdl = atoi(e);
    if (const char* e = getenv("CQ_MAX_STAGES")) v.max_stages = atoi(e);
    if (v.max_stages < 2) v.max_stages = 2;
    if (v.shape < 0 || v.shape >= N_SHAPES) v.shape = 0;
    return v;
  }();
  return k;
}

int align_up(int v, int a) { return (v + a - 1) / a * a; }

// Shared-memory plan for M activation rows; returns total bytes or -1 if it cannot fit.
int plan_smem(const cq_layer* L, int M, int grid, int max_smem, Shape sh, int target_kb, int max_stages,
              MatvecParams* p) {
  const uint32_t T = (uint32_t)L->n_sub * (uint32_t)L->n_gran;
  const uint32_t per = (T + grid - 1) / grid;
  const int max_pieces = (int)((per + L->n_gran - 1) / L->n_gran) + 1;
  const int mb = (M + 7) / 8;
  const int chunk_gran = sh.ncw * sh.gpw;
  p->nslot = max_pieces < 8 ? max_pieces : 8;
  p->max_cher = max_pieces;
  p->xs_stride = L->Kp + 8;
  p->xc_stride = L->Cp + 8;
  const int chunk = chunk_gran * L->gran_bytes;
  int off = 0;
  p->off_cher = off; off = align_up(off + p->max_cher * L->cher_bytes, 128);
  p->off_xs = off;   off = align_up(off + M * p->xs_stride * 2, 128);
  p->off_xc = off;   off = align_up(off + M * p->xc_stride * 2, 128);
  p->off_cidx = off; off = align_up(off + (L->Cp + 8) * 2, 128);
  p->off_corr = off; off = align_up(off + L->n_gran * L->sets * 8 * mb * 4, 128);
  // the octet-shift table is only needed while activations are staged: it shares the slots' space
  {
    const int slot_bytes = p->nslot * sh.ncw * M * 64, osh_bytes = (L->Kp / 8) * 4;
    p->off_slot = off; p->off_osh = off;
    off = align_up(off + (slot_bytes > osh_bytes ? slot_bytes : osh_bytes), 128);
  }
  p->off_pf = off;   off = align_up(off + 256 * 4, 128);
  p->off_bar = off;  off = align_up(off + (2 * 16 + 2) * 8, 128);
  p->off_ring = off;
  const int fixed = off;
  // Ring: with <= target_kb per CTA two launches overlap on one SM (the next layer prefetches its
  // weights while this one computes).  That only pays while the ring still holds enough bytes in
  // flight to cover HBM latency; otherwise take the whole SM.
  int budget = target_kb * 1024;
  if (budget - fixed < 64 * 1024) budget = max_smem;
  int stages = (budget - fixed) / chunk;
  if (stages > 16) stages = 16;
  if (stages > max_stages) stages = max_stages;
  const uint32_t max_chunks = per / chunk_gran + (uint32_t)max_pieces + 1;
  if ((uint32_t)stages > max_chunks) stages = (int)max_chunks;
  // The consumers run two ring stages ahead of their math: at least two stages are required.
  if (stages < 2) stages = 2;
  if (fixed + stages * chunk > max_smem) return -1;
  p->stages = stages;
  return fixed + stages * chunk;
}

}  // namespace

// Tracing: when a device buffer of 1024 x 16 uint64 is set, every CTA of the following matvec
// launches stores %globaltimer stamps of its phases there (slot meanings in cq_matvec_kernel).
extern "C" int cq_trace_set_timeline(void* device_buffer) {
  cq_g_timeline = (unsigned long long*)device_buffer;
  return CQ_OK;
}

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
  const Knobs kn = knobs();
  const Shape sh = SHAPES[kn.shape];
  const uint32_t T = (uint32_t)L->n_sub * (uint32_t)L->n_gran;
  int grid = di.sms < 1024 ? di.sms : 1024;
  if ((uint32_t)grid > T) grid = (int)T;

  MatvecParams p;
  int rows = M < 16 ? M : 16;
  int smem = -1;
  for (; rows >= 1; --rows) {
    smem = plan_smem(L, rows, grid, di.max_smem, sh, kn.smem_kb, kn.max_stages, &p);
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
  p.timeline = cq_g_timeline;
  p.M = rows; p.K = L->K; p.N = L->N; p.C = L->C; p.Cp = L->Cp; p.Kp = L->Kp;
  p.n_gran = L->n_gran; p.n_sub = L->n_sub; p.gran_bytes = L->gran_bytes; p.cher_bytes = L->cher_bytes;
  p.ldx = ldx; p.ldy = ldy; p.accumulate = accumulate;
  p.T = T;

  KernelFn fn = pick_kernel(kn.shape, L->bits, L->sets, (rows + 7) / 8);
  CQ_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3((sh.ncw + 1) * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = kn.pdl ? 1 : 0;
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
  const Knobs kn = knobs();
  const Shape sh = SHAPES[kn.shape];
  const uint32_t T = (uint32_t)L->n_sub * (uint32_t)L->n_gran;
  int grid = di.sms;
  if ((uint32_t)grid > T) grid = (int)T;

  // one launch must take all M rows: the array has room for one launch's partial sums only
  MatvecParams p;
  const int smem = plan_smem(L, M, grid, di.max_smem, sh, kn.smem_kb, kn.max_stages, &p);
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

  KernelFn fn = pick_kernel(kn.shape, L->bits, L->sets, (M + 7) / 8);
  CQ_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3((sh.ncw + 1) * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  CQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, fn, p));
  return CQ_OK;
}
