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
//    async copies (cp.async.bulk + mbarrier transaction counts), up to 8 granules
//    per copy.  It starts before the kernel waits for the previous kernel in the
//    stream (programmatic dependent launch): weights never depend on it.
//  * 8 consumer warps take the granules of a copy round-robin.  A lane reads its
//    16 (4-bit) or 24 (3-bit) bytes, turns codes into fp16 pairs with one
//    mask-or per pair (exponent trick) and one HFMA2, and feeds
//    mma.sync.m16n8k16 with the activations (staged once in shared memory in
//    compact order) as the B operand.  Group scales are applied per granule in
//    fp32.
//  * A range is walked from its last sub-tile to its first.  A sub-tile cut by a
//    range boundary is finished by the CTA that holds its end: CTAs holding an
//    earlier part post their fp32 partial to global scratch early in their walk,
//    the finishing CTA adds the partials in a fixed order late in its walk.  All
//    sums are therefore deterministic.  Every wait is bounded; running out sets
//    a bit in the status word instead of hanging.
#include "cq_common.cuh"

namespace {

constexpr int NCW = 8;                 // consumer warps
constexpr int NTHREADS = (NCW + 1) * 32;
constexpr int NCONS = NCW * 32;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

struct MatvecParams {
  const uint8_t* stream;
  const uint8_t* cstream;
  const uint16_t* perm;
  const uint16_t* cidx;
  const __half* x;
  __half* y;
  float* partial;      // [grid][256]
  uint32_t* flag;      // [grid]
  uint32_t* status;    // may be null
  int M, K, N, C, Cp, Kp, n_gran, n_sub, gran_bytes, cher_bytes;
  int ldx, ldy, accumulate;
  uint32_t T;          // total granules
  int stages, nslot, max_cher;
  // shared-memory offsets
  int off_ring, off_cher, off_xs, off_xc, off_slot, off_bar;
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t* status) {
  const uint32_t limit = *abort_flag ? 1u : WAIT_LIMIT;
  for (uint32_t it = 0; it < limit; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  *abort_flag = 1;
  if (status) atomicOr(status, 1u);
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
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
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// fp16x2 constants
constexpr uint32_t MAGIC = 0x64006400u;  // (1024, 1024)
// 4-bit: field at mantissa bit 2 -> 1024 + 4u, at bit 6 -> 1024 + 64u; u - 7.5 in one FMA
constexpr uint32_t S4_MUL_P2 = 0x34003400u;  // 0.25
constexpr uint32_t S4_ADD_P2 = 0xDC1EDC1Eu;  // -263.5
constexpr uint32_t S4_MUL_P6 = 0x24002400u;  // 1/64
constexpr uint32_t S4_ADD_P6 = 0xCDE0CDE0u;  // -23.5
// 3-bit: fields at mantissa bits 1, 4, 7; u - 3.5
constexpr uint32_t S3_MUL_P1 = 0x38003800u;  // 0.5
constexpr uint32_t S3_ADD_P1 = 0xE007E007u;  // -515.5
constexpr uint32_t S3_MUL_P4 = 0x2C002C00u;  // 1/16
constexpr uint32_t S3_ADD_P4 = 0xD438D438u;  // -67.5
constexpr uint32_t S3_MUL_P7 = 0x20002000u;  // 1/128
constexpr uint32_t S3_ADD_P7 = 0xC9C0C9C0u;  // -11.5

// One 4-bit stream word -> 4 fp16 pairs (codes (0,1), (2,3), (4,5), (6,7)), each u - 7.5.
__device__ __forceinline__ void dequant4(uint32_t w, uint32_t* out) {
  const uint32_t v1 = w << 2, v2 = w >> 6;
  out[0] = hfma2_u32((v1 & 0x003C003Cu) | MAGIC, S4_MUL_P2, S4_ADD_P2);
  out[1] = hfma2_u32((v1 & 0x03C003C0u) | MAGIC, S4_MUL_P6, S4_ADD_P6);
  out[2] = hfma2_u32((v2 & 0x003C003Cu) | MAGIC, S4_MUL_P2, S4_ADD_P2);
  out[3] = hfma2_u32((v2 & 0x03C003C0u) | MAGIC, S4_MUL_P6, S4_ADD_P6);
}

// Three 3-bit stream words of one row -> 16 fp16 pairs (codes (2q, 2q+1)), each u - 3.5.
__device__ __forceinline__ void dequant3(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t* out) {
  const uint32_t w[3] = {w0, w1, w2};
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const uint32_t v = w[i] >> 9;
    out[5 * i + 0] = hfma2_u32((w[i] & 0x000E000Eu) | MAGIC, S3_MUL_P1, S3_ADD_P1);
    out[5 * i + 1] = hfma2_u32((w[i] & 0x00700070u) | MAGIC, S3_MUL_P4, S3_ADD_P4);
    out[5 * i + 2] = hfma2_u32((w[i] & 0x03800380u) | MAGIC, S3_MUL_P7, S3_ADD_P7);
    out[5 * i + 3] = hfma2_u32((v & 0x000E000Eu) | MAGIC, S3_MUL_P1, S3_ADD_P1);
    out[5 * i + 4] = hfma2_u32((v & 0x00700070u) | MAGIC, S3_MUL_P4, S3_ADD_P4);
  }
  uint32_t r = ((w0 << 1) & 0x00020002u) | MAGIC;
  r |= (w1 << 2) & 0x00040004u;
  r |= (w2 << 3) & 0x00080008u;
  out[15] = hfma2_u32(r, S3_MUL_P1, S3_ADD_P1);
}

template <int BITS, int SETS, int MB>
__global__ void __launch_bounds__(NTHREADS, 1) cq_matvec_kernel(const MatvecParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t grid = gridDim.x, cta = blockIdx.x;
  const uint32_t ga = (uint32_t)(((uint64_t)p.T * cta) / grid);
  const uint32_t gb = (uint32_t)(((uint64_t)p.T * (cta + 1)) / grid);
  const uint32_t NG = (uint32_t)p.n_gran;
  const uint32_t GB = (uint32_t)p.gran_bytes;

  const uint32_t bar_base = smem_u32(smem + p.off_bar);
  const int S = p.stages;
  // barriers: full[s] at bar_base + 8 s, empty[s] at bar_base + 8 (S + s), cherry at 8 * 2S
  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_base + 8 * s, 1);
      mbar_init(bar_base + 8 * (S + s), NCW);
    }
    mbar_init(bar_base + 16 * S, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  // Let the next kernel in the stream start its own prologue and weight prefetch.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (ga >= gb) return;  // (host launches grid <= T, so this does not happen)

  const uint32_t j_hi = (gb - 1) / NG, j_lo = ga / NG;
  const int npieces = (int)(j_hi - j_lo + 1);
  const uint32_t jc_lo = (ga + NG - 1) / NG;           // first sub-tile whose start is in range
  const int ncher = (p.Cp > 0 && j_hi >= jc_lo) ? (int)(j_hi - jc_lo + 1) : 0;

  // ------------------------------------------------------------------ producer
  if (warp == NCW) {
    if (lane == 0) {
      if (ncher > 0) {
        const uint32_t bytes = (uint32_t)ncher * (uint32_t)p.cher_bytes;
        mbar_expect_tx(bar_base + 16 * S, bytes);
        bulk_g2s(smem_u32(smem + p.off_cher), p.cstream + (size_t)jc_lo * p.cher_bytes, bytes,
                 bar_base + 16 * S);
      }
      uint32_t cc = 0;
      for (int i = 0; i < npieces; ++i) {
        const uint32_t j = j_hi - i;
        const uint32_t start = max(ga, j * NG), end = min(gb, (j + 1) * NG);
        for (uint32_t q0 = start; q0 < end; q0 += NCW, ++cc) {
          const uint32_t len = min((uint32_t)NCW, end - q0);
          const uint32_t s = cc % S;
          if (cc >= (uint32_t)S) mbar_wait(bar_base + 8 * (S + s), ((cc / S) - 1) & 1, &s_abort, p.status);
          mbar_expect_tx(bar_base + 8 * s, len * GB);
          bulk_g2s(smem_u32(smem + p.off_ring) + s * NCW * GB, p.stream + (size_t)q0 * GB, len * GB,
                   bar_base + 8 * s);
        }
      }
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  // Everything below may read what the previous kernel in the stream wrote.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  __half* xs = reinterpret_cast<__half*>(smem + p.off_xs);
  __half* xc = reinterpret_cast<__half*>(smem + p.off_xc);
  for (int idx = tid; idx < p.M * p.Kp; idx += NCONS) {
    const int m = idx / p.Kp, k = idx - m * p.Kp;
    const uint32_t o = p.perm[k];
    xs[m * p.xs_stride + k] = (o != CQ_PAD_COL) ? p.x[(size_t)m * p.ldx + o] : __float2half(0.f);
  }
  for (int idx = tid; idx < p.M * p.Cp; idx += NCONS) {
    const int m = idx / p.Cp, c = idx - m * p.Cp;
    const uint32_t o = p.cidx[c];
    xc[m * p.xc_stride + c] = (o != CQ_PAD_COL) ? p.x[(size_t)m * p.ldx + o] : __float2half(0.f);
  }
  bar_consumers();

  const int g = lane >> 2, t = lane & 3;
  float4* slots = reinterpret_cast<float4*>(smem + p.off_slot);
  const uint8_t* ring = smem + p.off_ring;
  const uint8_t* cher = smem + p.off_cher;

  float tot[MB][4];
#pragma unroll
  for (int b = 0; b < MB; ++b)
#pragma unroll
    for (int r = 0; r < 4; ++r) tot[b][r] = 0.f;

  bool xrow_ok[MB];
  const __half* xrow[MB];
  const __half* xcrow[MB];
#pragma unroll
  for (int b = 0; b < MB; ++b) {
    const int m = 8 * b + g;
    xrow_ok[b] = m < p.M;
    xrow[b] = xs + (xrow_ok[b] ? m : 0) * p.xs_stride + 16 * t;
    xcrow[b] = xc + (xrow_ok[b] ? m : 0) * p.xc_stride + 2 * t;
  }

  uint32_t cc = 0, qrun = 0;
  int pending = 0;
  bool cher_ready = false;

  for (int i = 0; i < npieces; ++i) {
    const uint32_t j = j_hi - i;
    const uint32_t sub0 = j * NG;
    const uint32_t start = max(ga, sub0), end = min(gb, sub0 + NG);
    for (uint32_t q0 = start; q0 < end; q0 += NCW, ++cc) {
      const uint32_t len = min((uint32_t)NCW, end - q0);
      const uint32_t s = cc % S;
      mbar_wait(bar_base + 8 * s, (cc / S) & 1, &s_abort, p.status);
      const uint32_t o = ((uint32_t)warp - qrun) & (NCW - 1);
      qrun += len;
      if (o < len) {
        const uint32_t gi = q0 + o - sub0;               // granule inside the sub-tile
        const uint8_t* gran = ring + (size_t)s * NCW * GB + (size_t)o * GB;
        const __half* sc = reinterpret_cast<const __half*>(gran + 256 * BITS);
        float acc[MB][4];
#pragma unroll
        for (int b = 0; b < MB; ++b)
#pragma unroll
          for (int r = 0; r < 4; ++r) acc[b][r] = 0.f;

        uint32_t A0[16], A1[16];  // fp16 pairs of rows g and g+8 (8 per 64-column half)
        if (BITS == 4) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 w = *reinterpret_cast<const uint4*>(gran + h * 512 + lane * 16);
            dequant4(w.x, A0 + 8 * h);
            dequant4(w.y, A0 + 8 * h + 4);
            dequant4(w.z, A1 + 8 * h);
            dequant4(w.w, A1 + 8 * h + 4);
          }
        } else {
          const uint2* wp = reinterpret_cast<const uint2*>(gran + lane * 24);
          const uint2 u0 = wp[0], u1 = wp[1], u2 = wp[2];
          dequant3(u0.x, u0.y, u1.x, A0);
          dequant3(u1.y, u2.x, u2.y, A1);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int b = 0; b < MB; ++b) {
            uint4 xa = make_uint4(0, 0, 0, 0), xb = make_uint4(0, 0, 0, 0);
            if (xrow_ok[b]) {
              const uint4* xp = reinterpret_cast<const uint4*>(xrow[b] + gi * 128 + h * 64);
              xa = xp[0];
              xb = xp[1];
            }
            const uint32_t X[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
            for (int m = 0; m < 4; ++m)
              mma16816(acc[b], A0[8 * h + 2 * m], A1[8 * h + 2 * m], A0[8 * h + 2 * m + 1],
                       A1[8 * h + 2 * m + 1], X[2 * m], X[2 * m + 1]);
          }
          if (SETS == 2 || h == 1) {
            const int sp = (SETS == 2) ? h : 0;
            const float s0 = __half2float(sc[sp * 16 + g]), s1 = __half2float(sc[sp * 16 + g + 8]);
#pragma unroll
            for (int b = 0; b < MB; ++b) {
              tot[b][0] += s0 * acc[b][0];
              tot[b][1] += s0 * acc[b][1];
              tot[b][2] += s1 * acc[b][2];
              tot[b][3] += s1 * acc[b][3];
              acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.f;
            }
          }
        }
        // The granule that starts a sub-tile also adds the sub-tile's fp16 cherry columns.
        if (gi == 0 && p.Cp > 0) {
          if (!cher_ready) {
            mbar_wait(bar_base + 16 * S, 0, &s_abort, p.status);
            cher_ready = true;
          }
          const uint8_t* blk = cher + (size_t)(j - jc_lo) * p.cher_bytes;
          for (int jj = 0; jj < p.Cp / 16; ++jj) {
            const uint4 a = *reinterpret_cast<const uint4*>(blk + jj * 512 + lane * 16);
#pragma unroll
            for (int b = 0; b < MB; ++b) {
              uint32_t b0 = 0, b1 = 0;
              if (xrow_ok[b]) {
                b0 = *reinterpret_cast<const uint32_t*>(xcrow[b] + 16 * jj);
                b1 = *reinterpret_cast<const uint32_t*>(xcrow[b] + 16 * jj + 8);
              }
              mma16816(tot[b], a.x, a.y, a.z, a.w, b0, b1);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_base + 8 * (S + s));
    }

    // ---- end of piece i: park this warp's partial
    {
      float4* dst = slots + ((size_t)((i % p.nslot) * NCW + warp) * MB) * 32 + lane;
#pragma unroll
      for (int b = 0; b < MB; ++b) {
        dst[b * 32] = make_float4(tot[b][0], tot[b][1], tot[b][2], tot[b][3]);
        tot[b][0] = tot[b][1] = tot[b][2] = tot[b][3] = 0.f;
      }
    }
    ++pending;
    const bool post_now = (i == 0) && (end < sub0 + NG);   // piece 0 ends before its sub-tile does
    if (!(post_now || pending == p.nslot || i == npieces - 1)) continue;

    // ---- emit the pending pieces
    bar_consumers();
    uint32_t reset_lo = 1, reset_hi = 0;    // flags to clear afterwards (finishing CTA only)
    bool posted = false;
    for (int ii = i - pending + 1; ii <= i; ++ii) {
      const uint32_t jj = j_hi - ii;
      const uint32_t s0g = jj * NG;
      const uint32_t pstart = max(ga, s0g), pend = min(gb, s0g + NG);
      const int m = tid >> 4, r = tid & 15;
      float v = 0.f;
      if (m < p.M) {
        const int b = m >> 3, col = m & 7;
        const int ln = (r & 7) * 4 + (col >> 1);
        const int reg = (r >> 3) * 2 + (col & 1);
        const float* sl = reinterpret_cast<const float*>(slots + ((size_t)((ii % p.nslot) * NCW) * MB + b) * 32 + ln) + reg;
#pragma unroll
        for (int w = 0; w < NCW; ++w) v += sl[(size_t)w * MB * 32 * 4];
      }
      if (pend < s0g + NG) {
        // an earlier part of a cut sub-tile: hand the partial to the CTA that holds its end
        p.partial[(size_t)cta * 256 + tid] = v;
        posted = true;
      } else {
        if (pstart > s0g) {
          const uint32_t c_first = (uint32_t)((((uint64_t)s0g + 1) * grid - 1) / p.T);
          reset_lo = c_first;
          reset_hi = cta - 1;
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
            v += __ldcg(p.partial + (size_t)c * 256 + tid);
          }
        }
        const int n = (int)jj * 16 + r;
        if (m < p.M && n < p.N) {
          __half* yp = p.y + (size_t)m * p.ldy + n;
          if (p.accumulate) v += __half2float(*yp);
          *yp = __float2half(v);
        }
      }
    }
    bar_consumers();
    if (tid == 0) {
      if (posted) {
        __threadfence();
        st_release(p.flag + cta, 1u);
      }
      for (uint32_t c = reset_lo; c <= reset_hi && reset_lo <= reset_hi; ++c) p.flag[c] = 0u;
    }
    pending = 0;
  }
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
    cache[dev].max_smem = (int)prop.sharedMemPerBlockOptin;
    cache[dev].ok = true;
  }
  return cache[dev];
}

typedef void (*KernelFn)(const MatvecParams);

KernelFn pick_kernel(int bits, int sets, int mb) {
  if (bits == 4) {
    if (sets == 1) return mb == 1 ? cq_matvec_kernel<4, 1, 1> : cq_matvec_kernel<4, 1, 2>;
    return mb == 1 ? cq_matvec_kernel<4, 2, 1> : cq_matvec_kernel<4, 2, 2>;
  }
  if (sets == 1) return mb == 1 ? cq_matvec_kernel<3, 1, 1> : cq_matvec_kernel<3, 1, 2>;
  return mb == 1 ? cq_matvec_kernel<3, 2, 1> : cq_matvec_kernel<3, 2, 2>;
}

int align_up(int v, int a) { return (v + a - 1) / a * a; }

// Shared-memory plan for M activation rows; returns total bytes or -1 if it cannot fit.
int plan_smem(const cq_layer* L, int M, int grid, int max_smem, MatvecParams* p) {
  const uint32_t T = (uint32_t)L->n_sub * (uint32_t)L->n_gran;
  const uint32_t per = (T + grid - 1) / grid;
  const int max_pieces = (int)((per + L->n_gran - 1) / L->n_gran) + 1;
  const int mb = (M + 7) / 8;
  p->nslot = max_pieces < 8 ? max_pieces : 8;
  p->max_cher = max_pieces;
  p->xs_stride = L->Kp + 8;
  p->xc_stride = L->Cp + 8;
  const int chunk = NCW * L->gran_bytes;
  int off = 0;
  p->off_cher = off; off = align_up(off + p->max_cher * L->cher_bytes, 128);
  p->off_xs = off;   off = align_up(off + M * p->xs_stride * 2, 128);
  p->off_xc = off;   off = align_up(off + M * p->xc_stride * 2, 128);
  p->off_slot = off; off = align_up(off + p->nslot * NCW * mb * 512, 128);
  p->off_bar = off;  off = align_up(off + (2 * 16 + 1) * 8, 128);
  p->off_ring = off;
  const int fixed = off;
  // Ring: aim at <= ~112 KB per CTA so two launches can overlap on one SM, but never
  // fewer than 3 stages; never more than 16.
  const int target = 112 * 1024;
  int stages = (target - fixed) / chunk;
  if (stages < 3) stages = 3;
  if (stages > 16) stages = 16;
  const uint32_t max_chunks = per / NCW + (uint32_t)max_pieces + 1;
  if ((uint32_t)stages > max_chunks) stages = (int)max_chunks;
  if (stages < 1) stages = 1;
  while (stages > 1 && fixed + stages * chunk > max_smem) --stages;
  if (fixed + stages * chunk > max_smem) return -1;
  p->stages = stages;
  return fixed + stages * chunk;
}

}  // namespace

extern "C" size_t cq_scratch_bytes(void) {
  // up to 1024 CTAs: 256 floats of partial + one flag each
  return (size_t)1024 * 256 * sizeof(float) + 1024 * sizeof(uint32_t);
}

// Launches over at most `rows` activation rows at a time; the caller (cq_layer_matvec)
// splits larger batches.
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
  int smem = -1;
  for (; rows >= 1; --rows) {
    smem = plan_smem(L, rows, grid, di.max_smem, &p);
    if (smem >= 0) break;
  }
  if (smem < 0) return CQ_ERR_TOO_LARGE;
  const uint8_t* blob = (const uint8_t*)L->blob;
  p.stream = blob + L->off_stream;
  p.cstream = blob + L->off_cherry;
  p.perm = (const uint16_t*)(blob + L->off_perm);
  p.cidx = (const uint16_t*)(blob + L->off_cidx);
  p.x = x; p.y = y;
  p.partial = (float*)scratch;
  p.flag = (uint32_t*)((uint8_t*)scratch + (size_t)1024 * 256 * sizeof(float));
  p.status = status;
  p.M = rows; p.K = L->K; p.N = L->N; p.C = L->C; p.Cp = L->Cp; p.Kp = L->Kp;
  p.n_gran = L->n_gran; p.n_sub = L->n_sub; p.gran_bytes = L->gran_bytes; p.cher_bytes = L->cher_bytes;
  p.ldx = ldx; p.ldy = ldy; p.accumulate = accumulate;
  p.T = T;

  KernelFn fn = pick_kernel(L->bits, L->sets, (rows + 7) / 8);
  CQ_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(NTHREADS);
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
