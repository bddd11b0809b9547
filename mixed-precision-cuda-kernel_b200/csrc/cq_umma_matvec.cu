// Decode matvec (1..16 activation rows) of a tile-layout CherryQ layer on the 5th-generation
// tensor cores: tcgen05.mma with the weights as the A operand in TENSOR MEMORY and the
// activations as the B operand in shared memory.
//
//   y[m, n] (+)= sum_k' (u[k', n] - off) * s[group(k'), n] * x[m, orig(k')]
//              + sum_c  cherry_weight[c, n] * x[m, idx[c]]
// (what the reference kernels csrc/quant_cuda_kernel.cu:718-835, :558-672, :316-438 compute).
//
// Why tensor memory: a 4-bit weight costs 0.75 integer instructions to turn into an fp16 operand,
// and that is all a thread does here.  One thread owns one weight ROW (= one TMEM lane): it reads
// the row's packed words from shared memory, ANDs code fields into the bit pattern of fp16
// 1024.0 (see "decode" below), and stores the fp16 pairs straight into TMEM with tcgen05.st.
// No mma.sync fragments, no B-operand loads, no per-granule floating-point epilogue in the hot
// path: the MMA is issued asynchronously by one thread and accumulates a whole 128-column group
// in TMEM, which the row's thread reads back once per group to apply the group's scale.
//
// Warp roles (one CTA per SM, two CTAs of consecutive launches may share an SM):
//   decode warps   NGRP groups of 4 warps; group g takes items n = g, g + NGRP, ... of the CTA's
//                  item sequence; thread r of a group owns row r of the 128-row tile
//   MMA warp       one lane issues tcgen05.mma / tcgen05.commit; the warp owns the TMEM allocation
//   producer warp  one lane streams the items (cp.async.bulk) into a shared-memory ring; later
//                  prefetches partial sums of a tile that earlier CTAs started
//   stager warps   gather the activations of the columns the CTA needs, pre-scale them, write
//                  them in the canonical K-major UMMA layout, and sum the per-group corrections
//
// Work distribution: the layer is a flat sequence of items (per 128-row tile: its cherry items,
// then its granules of 128 columns); CTA c owns items [T*c/grid, T*(c+1)/grid).  Tiles cut by a
// range boundary are finished by the CTA that holds their end, from partial sums the earlier
// CTAs post to global scratch early in their walk (ranges are walked last tile first).
// All sums have a fixed order (deterministic); every wait is bounded and reports into a status
// word instead of hanging.
#include <cstdlib>

#include "cq_tile.cuh"

extern unsigned long long* cq_g_timeline;

namespace {

constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr int NA = 3;          // A slots in TMEM (64 columns each)
constexpr int A_COLS = 64;
constexpr int D_BASE = NA * A_COLS;   // 64 columns of accumulators behind the A slots
constexpr int TMEM_COLS = 256;
constexpr int WIN_GRAN = 4;    // granules per activation window
constexpr int NCORR = 32;      // correction ring (items)
constexpr int MAX_STAGES = 14;
constexpr int NXMAX = 3;

struct UmmaParams {
  const uint8_t* stream;
  const uint16_t* cidx;
  const uint32_t* osh;
  const __half* x;
  __half* y;
  float* partial;      // [grid][16][128]
  uint32_t* flag;      // [grid]
  uint32_t* status;
  unsigned long long* timeline;   // may be null: [grid][64] %globaltimer stamps (tracing)
  int M, K, N, C, Cp, Kp, n_gran, n_tile, n_cher, gran_bytes, tile_bytes, ipt;
  int ldx, ldy, accumulate;
  uint32_t T;          // total items
  int stages, nx, stage_bytes, xwin_bytes, sbo16, xc_sbo16;
  int off_ring, off_xwin, off_xc, off_corr, off_cidx, off_osh, off_slot, off_pf, off_bar, off_misc;
};

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
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
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                            uint32_t* status, uint32_t code) {
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
  if (status) atomicOr(status, code);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t* status,
                                          uint32_t code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status, code);
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
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
__device__ __forceinline__ void named_bar(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem_d] (+)= A[tmem_a] * B[desc_b], M = 128, N = 16, K = 16, fp16 inputs, fp32 accumulate
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(acc), "r"(0u) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                 "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t addr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t addr, float* v) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(addr) : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tstamp(const UmmaParams& p, int slot) {
  if (p.timeline) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.timeline[(size_t)blockIdx.x * 64 + slot] = t;
  }
}

// ------------------------------------------------------------------ decode
// OR-ing a code field that sits at mantissa bit p into the bit pattern of 1024.0 gives the fp16
// number 1024 + 2^p * u.  The activation that meets this code in the MMA is pre-multiplied by
// 2^(c-p) when it is staged, so the product is 2^c * (B + u) * x with B = 2^(10-p); the excess
// (B + off) * x, summed per group while staging ("corr"), is removed in fp32 when the group's
// scale is applied:  y += s * (acc * 2^-c - corr).  p depends on the column's position only.
constexpr uint32_t MAGIC = 0x64006400u;
template <int BITS> struct Fold;
template <> struct Fold<4> { static constexpr int C_EXP = 2; static constexpr float OFF = 7.5f; };
template <> struct Fold<3> { static constexpr int C_EXP = 1; static constexpr float OFF = 3.5f; };
// p of compact column k' (4-bit: pair (k' >> 1) even -> 2, odd -> 6; 3-bit: pair q = (k' % 32) >> 1
// -> 1, 4, 7, 4, 7 by q % 5, pair 15 -> 7)
template <int BITS>
__device__ __forceinline__ int fold_p_pair(int q) {
  if (BITS == 4) return (q & 1) ? 6 : 2;
  const int r = q % 5;
  return q == 15 ? 7 : (r == 0 ? 1 : ((r & 1) ? 4 : 7));
}
__device__ __forceinline__ void decode4(uint32_t w, uint32_t* out) {
  const uint32_t v1 = w << 2, v2 = w >> 6;
  out[0] = (v1 & 0x003C003Cu) | MAGIC;
  out[1] = (v1 & 0x03C003C0u) | MAGIC;
  out[2] = (v2 & 0x003C003Cu) | MAGIC;
  out[3] = (v2 & 0x03C003C0u) | MAGIC;
}
__device__ __forceinline__ void decode3(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t* out) {
  const uint32_t w[3] = {w0, w1, w2};
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const uint32_t v = w[i] >> 6;
    out[5 * i + 0] = (w[i] & 0x000E000Eu) | MAGIC;
    out[5 * i + 1] = (w[i] & 0x00700070u) | MAGIC;
    out[5 * i + 2] = (w[i] & 0x03800380u) | MAGIC;
    out[5 * i + 3] = (v & 0x00700070u) | MAGIC;
    out[5 * i + 4] = (v & 0x03800380u) | MAGIC;
  }
  uint32_t r = ((w0 << 7) & 0x00800080u) | MAGIC;
  r |= (w1 << 8) & 0x01000100u;
  r |= (w2 << 9) & 0x02000200u;
  out[15] = r;
}

// Shared-memory matrix descriptor of a K-major, unswizzled operand: rows of a core matrix 16 B
// apart, the two 8-column halves of a 16-column step `lbo` bytes apart, 8-row groups `sbo` apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo16, uint32_t sbo16) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)lbo16 << 16) | ((uint64_t)sbo16 << 32) | ((uint64_t)1 << 46);
}

// The CTA's walk over its items: tiles from last to first, items of a tile in order.
struct Walk {
  uint32_t ia, ib, ipt;
  int piece;           // piece index (0 = last tile of the range)
  uint32_t tile, start, end, cur;
  __device__ __forceinline__ void init(uint32_t a, uint32_t b, uint32_t ipt_) {
    ia = a; ib = b; ipt = ipt_;
    piece = 0;
    tile = (ib - 1) / ipt;
    set_piece();
  }
  __device__ __forceinline__ void set_piece() {
    start = max(ia, tile * ipt);
    end = min(ib, (tile + 1) * ipt);
    cur = start;
  }
  __device__ __forceinline__ bool done() const { return cur >= end && start <= ia; }
  // advance to the next item; returns false when the walk is over
  __device__ __forceinline__ bool next() {
    ++cur;
    if (cur < end) return true;
    if (start <= ia) return false;
    --tile; ++piece;
    set_piece();
    return true;
  }
};

template <int BITS, int SETS, int MB, int NGRP>
__global__ void __launch_bounds__((NGRP * 4 + 4) * 32, 1) cq_umma_matvec_kernel(const UmmaParams p) {
  constexpr int NDEC = NGRP * 4;                  // decode warps
  constexpr int W_MMA = NDEC, W_PROD = NDEC + 1, W_STG = NDEC + 2;
  constexpr int D_COLS = 16 * SETS;               // accumulator columns per item
  constexpr int ND = 64 / D_COLS;                 // accumulator buffers
  constexpr int MT = 8 * MB;                      // activation rows handled (padded)
  constexpr int CE = Fold<BITS>::C_EXP;
  constexpr uint32_t IDESC = (1u << 4) | (2u << 17) | (8u << 24);   // F32 acc, F16 A/B, K-major, N=16, M=128
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_abort;
  __shared__ uint32_t s_tmem;
  __shared__ int s_slotcnt[2];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t grid = gridDim.x, cta = blockIdx.x;
  const uint32_t ia = (uint32_t)(((uint64_t)p.T * cta) / grid);
  const uint32_t ib = (uint32_t)(((uint64_t)p.T * (cta + 1)) / grid);
  const uint32_t IPT = (uint32_t)p.ipt, NCH = (uint32_t)p.n_cher;
  const uint32_t S = (uint32_t)p.stages, NX = (uint32_t)p.nx;

  // barrier table
  const uint32_t bar0 = smem_u32(smem + p.off_bar);
  auto B_WFULL = [&](uint32_t s) { return bar0 + 8 * s; };
  auto B_WEMPTY = [&](uint32_t s) { return bar0 + 8 * (MAX_STAGES + s); };
  auto B_AFULL = [&](uint32_t a) { return bar0 + 8 * (2 * MAX_STAGES + a); };
  auto B_AEMPTY = [&](uint32_t a) { return bar0 + 8 * (2 * MAX_STAGES + NA + a); };
  auto B_DFULL = [&](uint32_t d) { return bar0 + 8 * (2 * MAX_STAGES + 2 * NA + d); };
  auto B_DEMPTY = [&](uint32_t d) { return bar0 + 8 * (2 * MAX_STAGES + 2 * NA + 4 + d); };
  auto B_XFULL = [&](uint32_t x) { return bar0 + 8 * (2 * MAX_STAGES + 2 * NA + 8 + x); };
  auto B_XEMPTY = [&](uint32_t x) { return bar0 + 8 * (2 * MAX_STAGES + 2 * NA + 8 + NXMAX + x); };
  const uint32_t B_XC = bar0 + 8 * (2 * MAX_STAGES + 2 * NA + 8 + 2 * NXMAX);
  const uint32_t B_PF = B_XC + 8;

  if (tid == 0) {
    tstamp(p, 0);
    s_abort = 0;
    s_slotcnt[0] = s_slotcnt[1] = 0;
    for (uint32_t s = 0; s < S; ++s) { mbar_init(B_WFULL(s), 1); mbar_init(B_WEMPTY(s), 4); }
    for (uint32_t a = 0; a < NA; ++a) { mbar_init(B_AFULL(a), 4); mbar_init(B_AEMPTY(a), 1); }
    for (uint32_t d = 0; d < 4; ++d) { mbar_init(B_DFULL(d), 1); mbar_init(B_DEMPTY(d), 4); }
    for (uint32_t x = 0; x < NXMAX; ++x) { mbar_init(B_XFULL(x), 1); mbar_init(B_XEMPTY(x), 1); }
    mbar_init(B_XC, 2);
    mbar_init(B_PF, 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == W_MMA) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  if (tid == 0) tstamp(p, 1);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const bool has_work = ia < ib;
  float* corr = reinterpret_cast<float*>(smem + p.off_corr);           // [NCORR][SETS][16]

  if (has_work && warp == W_PROD) {
    // ================================================================ producer
    if (lane == 0) {
      const uint32_t ring = smem_u32(smem + p.off_ring);
      Walk w; w.init(ia, ib, IPT);
      uint32_t n = 0;
      do {
        const uint32_t j = w.cur - w.tile * IPT;
        const uint32_t bytes = j < NCH ? (uint32_t)CQT_CHER_BYTES : (uint32_t)p.gran_bytes;
        const size_t off = (size_t)w.tile * p.tile_bytes +
                           (j < NCH ? (size_t)j * CQT_CHER_BYTES : (size_t)NCH * CQT_CHER_BYTES + (size_t)(j - NCH) * p.gran_bytes);
        const uint32_t s = n % S;
        if (n >= S) mbar_wait(B_WEMPTY(s), ((n / S) - 1) & 1, &s_abort, p.status, 1u);
        if (n == 0) tstamp(p, 12);
        mbar_expect_tx(B_WFULL(s), bytes);
        bulk_g2s(ring + s * (uint32_t)p.stage_bytes, p.stream + off, bytes, B_WFULL(s));
        ++n;
      } while (w.next());
      tstamp(p, 13);
    }
    // Partial sums of the tile at the head of this range that earlier CTAs started: they were
    // posted early in those CTAs' walks.  The scratch may still hold the previous launch's flags
    // until that launch has completed, so wait for it first.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
      float* pf = reinterpret_cast<float*>(smem + p.off_pf);            // [MT][128]
      const uint32_t t_lo = ia / IPT;
      const uint32_t t0 = t_lo * IPT;
      constexpr int PER = MT * 128 / 32;
      float v[PER];
#pragma unroll
      for (int e = 0; e < PER; ++e) v[e] = 0.f;
      if (ia > t0 && ib >= t0 + IPT) {
        const uint32_t c_first = (uint32_t)((((uint64_t)t0 + 1) * grid - 1) / p.T);
        for (uint32_t c = c_first; c < cta; ++c) {
          bool ok = false;
          const uint32_t limit = s_abort ? 1u : WAIT_LIMIT;
          for (uint32_t it = 0; it < limit; ++it) {
            if (ld_acquire(p.flag + c) != 0) { ok = true; break; }
            __nanosleep(64);
          }
          if (!ok) { s_abort = 1; if (p.status) atomicOr(p.status, 2u); }
#pragma unroll
          for (int e = 0; e < PER; ++e) v[e] += __ldcg(p.partial + (size_t)c * 2048 + e * 32 + lane);
        }
      }
#pragma unroll
      for (int e = 0; e < PER; ++e) pf[e * 32 + lane] = v[e];
      mbar_arrive(B_PF);
    }
  } else if (has_work && warp >= W_STG) {
    // ================================================================ stagers (64 threads)
    const int st = tid - W_STG * 32;
    uint16_t* cidx_s = reinterpret_cast<uint16_t*>(smem + p.off_cidx);
    uint32_t* osh_s = reinterpret_cast<uint32_t*>(smem + p.off_osh);
    uint8_t* xwin = smem + p.off_xwin;
    uint8_t* xcb = smem + p.off_xc;
    // layer constants and zero fill (rows past M of every 8-row group stay zero for good)
    for (int c = st; c < p.Cp; c += 64) cidx_s[c] = p.cidx[c];
    for (int o = st; o < (p.Kp >> 3); o += 64) osh_s[o] = p.osh[o];
    for (int i = st; i < (int)(NX * p.xwin_bytes) / 16; i += 64) reinterpret_cast<uint4*>(xwin)[i] = make_uint4(0, 0, 0, 0);
    for (int i = st; i < (p.n_cher * 256 * MB) / 16; i += 64) reinterpret_cast<uint4*>(xcb)[i] = make_uint4(0, 0, 0, 0);
    for (int i = st; i < NCORR * SETS * 16; i += 64) corr[i] = 0.f;
    named_bar(2, 64);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (st == 0) tstamp(p, 2);

    // activations of the cherry columns, unscaled: [item j][half c][row r][8 fp16] (+ row group)
    for (int idx = st; idx < p.M * p.Cp; idx += 64) {
      const int m = idx / p.Cp, c = idx - m * p.Cp;
      const uint32_t o = cidx_s[c];
      const __half v = (o != CQ_PAD_COL) ? p.x[(size_t)m * p.ldx + o] : __float2half(0.f);
      const int j = c >> 4, cc = (c >> 3) & 1, e = c & 7;
      reinterpret_cast<__half*>(xcb + (m >> 3) * (p.xc_sbo16 << 4) + j * 256 + cc * 128 + (m & 7) * 16)[e] = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive(B_XC);
    if (st == 0) tstamp(p, 3);

    // Windows of up to WIN_GRAN granules, in the order the MMA warp consumes them.  The two stager
    // warps take alternate windows, so that two windows' trips to L2 overlap; a lane stages the
    // octets `lane` and `lane + 32` of its window (16 octets per granule).
    const int sw = warp - W_STG;
    Walk w; w.init(ia, ib, IPT);
    uint32_t n = 0, wn = 0;
    bool more = true;
    while (more) {
      const uint32_t j = w.cur - w.tile * IPT;
      if (j < NCH) { more = w.next(); ++n; continue; }
      // a window starts here: granules g0 .. g0 + len - 1 of this tile, items n .. n + len - 1
      const uint32_t g0 = j - NCH;
      const uint32_t len = min((uint32_t)WIN_GRAN, w.end - w.cur);
      if ((int)(wn & 1) == sw) {
        const uint32_t xs = wn % NX;
        uint8_t* win = xwin + (size_t)xs * p.xwin_bytes;
        bool waited = false;
        for (int m0 = 0; m0 < p.M; m0 += 2) {
          uint32_t v[2][2][4];
          uint32_t shv[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int oc = lane + 32 * h, gw = oc >> 4, oo = oc & 15;
            const int o = (int)(g0 + gw) * 16 + oo;
            shv[h] = ((uint32_t)gw < len) ? osh_s[o] : 0xFFFFFFFFu;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              v[u][h][0] = v[u][h][1] = v[u][h][2] = v[u][h][3] = 0u;
              const int m = m0 + u;
              if (m < p.M && shv[h] != 0xFFFFFFFFu) {
                const int lo0 = (int)(shv[h] & 0xFFFFu), lo7 = (int)(shv[h] >> 16);
                const __half* xr = p.x + (size_t)m * p.ldx;
                const int k0 = 8 * o;
                if (lo7 == lo0) {
                  const int src = k0 + lo0;
                  if ((src & 1) == 0 && (((uintptr_t)xr) & 3) == 0) {
                    const uint32_t* s32 = reinterpret_cast<const uint32_t*>(xr + src);
#pragma unroll
                    for (int i = 0; i < 4; ++i) v[u][h][i] = __ldg(s32 + i);
                  } else {
                    const unsigned short* s16 = reinterpret_cast<const unsigned short*>(xr + src);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                      v[u][h][i] = (uint32_t)__ldg(s16 + 2 * i) | ((uint32_t)__ldg(s16 + 2 * i + 1) << 16);
                  }
                } else {
                  unsigned short hh[8];
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    int lo = lo0, hi = lo7;
                    while (lo < hi) {
                      const int mid = (lo + hi) >> 1;
                      if ((int)cidx_s[mid] - mid <= k0 + i) lo = mid + 1; else hi = mid;
                    }
                    hh[i] = __ldg(reinterpret_cast<const unsigned short*>(xr + k0 + i + lo));
                  }
#pragma unroll
                  for (int i = 0; i < 4; ++i) v[u][h][i] = (uint32_t)hh[2 * i] | ((uint32_t)hh[2 * i + 1] << 16);
                }
              }
            }
          }
          // the slot is only needed now, after the loads are in flight
          if (!waited) {
            if (wn >= NX) mbar_wait(B_XEMPTY(xs), ((wn / NX) - 1) & 1, &s_abort, p.status, 4u);
            waited = true;
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int oc = lane + 32 * h, gw = oc >> 4, oo = oc & 15;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int m = m0 + u;
              // pair index of the octet's first pair: 4-bit (k' >> 1) parity only; 3-bit (k' % 32) >> 1
              const int q0 = (BITS == 4) ? 0 : 4 * (oo & 3);
              float acc = 0.f;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int pp = fold_p_pair<BITS>(q0 + i);
                const uint32_t sc16 = (uint32_t)((15 + CE - pp) << 10);
                const uint32_t scaled = hmul2_u32(v[u][h][i], sc16 | (sc16 << 16));
                const float coef = __int_as_float((127 + pp - CE) << 23) * ((float)(1 << (10 - pp)) + Fold<BITS>::OFF);
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&scaled));
                acc += (f.x + f.y) * coef;
                v[u][h][i] = scaled;
              }
              // 16 (8 for 64-wide groups) neighbouring lanes hold the octets of one group of one row
#pragma unroll
              for (int dlt = 1; dlt < 16 / SETS; dlt <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, dlt);
              if ((uint32_t)gw < len && m < p.M) {
                // B operand, K-major: [16-column step][column half][row of the 8-row group][8 fp16]
                uint8_t* dst = win + (m >> 3) * (p.sbo16 << 4) + (gw * 8 + (oo >> 1)) * 256 + (oo & 1) * 128 + (m & 7) * 16;
                *reinterpret_cast<uint4*>(dst) = make_uint4(v[u][h][0], v[u][h][1], v[u][h][2], v[u][h][3]);
                if ((oo & (16 / SETS - 1)) == 0) {
                  const int sp = (SETS == 2) ? (oo >> 3) : 0;
                  corr[(((n + gw) % NCORR) * SETS + sp) * 16 + m] = acc;
                }
              }
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) { mbar_arrive(B_XFULL(xs)); if (wn < 8) tstamp(p, 4 + wn); }
      }
      ++wn;
      for (uint32_t e = 0; e < len && more; ++e) { more = w.next(); ++n; }
    }
  } else if (has_work && warp == W_MMA) {
    // ================================================================ MMA issuer
    if (lane == 0) {
      const uint32_t xwin = smem_u32(smem + p.off_xwin), xcb = smem_u32(smem + p.off_xc);
      Walk w; w.init(ia, ib, IPT);
      uint32_t n = 0, wn = 0, in_win = 0, win_len = 0;
      bool xc_ready = false, more = true;
      while (more) {
        const uint32_t j = w.cur - w.tile * IPT;
        const uint32_t a = n % NA, d = n % ND;
        mbar_wait(B_AFULL(a), (n / NA) & 1, &s_abort, p.status, 8u);
        if (n >= ND) mbar_wait(B_DEMPTY(d), ((n / ND) - 1) & 1, &s_abort, p.status, 16u);
        const uint32_t ta = tmem + a * A_COLS, td = tmem + D_BASE + d * D_COLS;
        if (j < NCH) {
          if (!xc_ready) { mbar_wait(B_XC, 0, &s_abort, p.status, 32u); xc_ready = true; }
          tc_fence_after();
          umma_ts(td, ta, smem_desc(xcb + j * 256, 8, (uint32_t)p.xc_sbo16), IDESC, 0u);
        } else {
          if (in_win == 0) {
            win_len = min((uint32_t)WIN_GRAN, w.end - w.cur);
            mbar_wait(B_XFULL(wn % NX), (wn / NX) & 1, &s_abort, p.status, 64u);
          }
          tc_fence_after();
          const uint32_t base = xwin + (wn % NX) * (uint32_t)p.xwin_bytes + in_win * 8 * 256;
#pragma unroll
          for (uint32_t ks = 0; ks < 8; ++ks) {
            const uint32_t dcol = (SETS == 2) ? (ks >> 2) * 16 : 0;
            const uint32_t acc = (SETS == 2) ? ((ks & 3) != 0) : (ks != 0);
            umma_ts(td + dcol, ta + ks * 8, smem_desc(base + ks * 256, 8, (uint32_t)p.sbo16), IDESC, acc);
          }
          if (++in_win == win_len) {
            tc_commit(B_XEMPTY(wn % NX));
            in_win = 0;
            ++wn;
          }
        }
        tc_commit(B_AEMPTY(a));
        tc_commit(B_DFULL(d));
        if (n < 24) tstamp(p, 16 + n);
        ++n;
        more = w.next();
      }
    }
  } else if (has_work && warp < NDEC) {
    // ================================================================ decode groups
    const int grp = warp >> 2;
    const int row = (warp & 3) * 32 + lane;                 // row of the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint8_t* ring = smem + p.off_ring;
    float* slot = reinterpret_cast<float*>(smem + p.off_slot);          // [2][MT][128]
    const float* pf = reinterpret_cast<const float*>(smem + p.off_pf);
    const int gtid = tid - grp * 128;

    float tot[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) tot[m] = 0.f;
    int tot_piece = 0;                      // piece the accumulators in `tot` belong to

    // deferred epilogue of this group's previous item
    bool pend = false;
    uint32_t pend_n = 0;
    int pend_piece = 0;
    float pend_s0 = 0.f, pend_s1 = 0.f, pend_inv = 1.f;
    bool pend_corr = false;

    // Emits piece `pc` once every group has added its accumulators to the piece's slot, in group
    // order (fixed summation order).  The last group finishes the piece.
    auto flush_piece = [&](int pc) {
      const int sl = pc & 1;
      volatile int* cnt = &s_slotcnt[sl];
      // wait for my turn: groups add in order 0, 1, ..., NGRP-1
      {
        const uint32_t limit = s_abort ? 1u : WAIT_LIMIT;
        bool ok = false;
        for (uint32_t it = 0; it < limit; ++it) {
          if (*cnt == grp) { ok = true; break; }
          __nanosleep(32);
        }
        if (!ok) { s_abort = 1; if (p.status) atomicOr(p.status, 128u); }
      }
      float* s = slot + (size_t)sl * MT * 128;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m < p.M) {
          const float prev = (grp == 0) ? 0.f : s[m * 128 + row];
          s[m * 128 + row] = prev + tot[m];
        }
        tot[m] = 0.f;
      }
      __threadfence_block();
      named_bar(3 + grp, 128);
      if (grp < NGRP - 1) {
        if (gtid == 0) *cnt = grp + 1;
        return;
      }
      // ---- last group: finish the piece
      const uint32_t tile = (ib - 1) / IPT - (uint32_t)pc;
      const uint32_t t0 = tile * IPT;
      const uint32_t pstart = max(ia, t0), pend_i = min(ib, t0 + IPT);
      const int n_row = (int)tile * 128 + row;
      if (pend_i < t0 + IPT) {
        // an earlier part of a cut tile: hand the partial to the CTA that holds the tile's end
#pragma unroll
        for (int m = 0; m < MT; ++m)
          if (m < p.M) p.partial[(size_t)cta * 2048 + m * 128 + row] = s[m * 128 + row];
        __threadfence();
        named_bar(3 + grp, 128);
        if (gtid == 0) st_release(p.flag + cta, 1u);
      } else {
        const bool cut = pstart > t0;
        if (cut) mbar_wait(B_PF, 0, &s_abort, p.status, 256u);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (m < p.M && n_row < p.N) {
            float v = s[m * 128 + row];
            if (cut) v += pf[m * 128 + row];
            __half* yp = p.y + (size_t)m * p.ldy + n_row;
            if (p.accumulate) v += __half2float(*yp);
            *yp = __float2half(v);
          }
        }
        if (cut) {
          named_bar(3 + grp, 128);
          if (gtid == 0) {
            const uint32_t c_first = (uint32_t)((((uint64_t)t0 + 1) * grid - 1) / p.T);
            for (uint32_t c = c_first; c < cta; ++c) p.flag[c] = 0u;
          }
        }
      }
      named_bar(3 + grp, 128);
      if (gtid == 0) *cnt = 0;
    };

    auto epilogue = [&]() {
      // scale and add the accumulators of the pending item, then free its TMEM buffer
      const uint32_t d = pend_n % ND;
      if (pend_piece != tot_piece) {
        for (int pc = tot_piece; pc < pend_piece; ++pc) flush_piece(pc);
        tot_piece = pend_piece;
      }
      mbar_wait(B_DFULL(d), (pend_n / ND) & 1, &s_abort, p.status, 512u);
      tc_fence_after();
      float dv[SETS][MT];
#pragma unroll
      for (int sp = 0; sp < SETS; ++sp)
#pragma unroll
        for (int b = 0; b < MB; ++b)
          tmem_ld8(tmem + lane_addr + D_BASE + d * D_COLS + sp * 16 + b * 8, &dv[sp][b * 8]);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(B_DEMPTY(d));
      const float* cr = corr + (size_t)(pend_n % NCORR) * SETS * 16;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (pend_corr) {
          tot[m] += pend_s0 * (dv[0][m] * pend_inv - cr[m]);
          if (SETS == 2) tot[m] += pend_s1 * (dv[1][m] * pend_inv - cr[16 + m]);
        } else {
          tot[m] += dv[0][m];
        }
      }
      pend = false;
    };

    Walk w; w.init(ia, ib, IPT);
    uint32_t n = 0;
    bool more = true;
    int last_piece = 0;
    while (more) {
      last_piece = w.piece;
      if ((int)(n % NGRP) == grp) {
        const uint32_t j = w.cur - w.tile * IPT;
        const uint32_t s = n % S, a = n % NA;
        mbar_wait(B_WFULL(s), (n / S) & 1, &s_abort, p.status, 1024u);
        const uint8_t* item = ring + (size_t)s * p.stage_bytes;
        const bool cherry = j < NCH;
        constexpr int NW = 4 * BITS;
        uint4 raw[BITS];
        float s0 = 1.f, s1 = 1.f;
        if (cherry) {
          raw[0] = *reinterpret_cast<const uint4*>(item + row * 16);
          raw[1] = *reinterpret_cast<const uint4*>(item + 2048 + row * 16);
        } else {
#pragma unroll
          for (int q = 0; q < BITS; ++q) raw[q] = *reinterpret_cast<const uint4*>(item + q * 2048 + row * 16);
          const __half* sc = reinterpret_cast<const __half*>(item + 2048 * BITS);
          s0 = __half2float(sc[row]);
          if (SETS == 2) s1 = __half2float(sc[128 + row]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(B_WEMPTY(s));
        if (n >= NA) mbar_wait(B_AEMPTY(a), ((n / NA) - 1) & 1, &s_abort, p.status, 2048u);
        tc_fence_after();
        const uint32_t ta = tmem + lane_addr + a * A_COLS;
        if (cherry) {
          const uint32_t v[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
          tmem_st8(ta, v);
        } else {
          const uint32_t* wds = reinterpret_cast<const uint32_t*>(raw);
          (void)NW;
          if (BITS == 4) {
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              uint32_t v[16];
#pragma unroll
              for (int e = 0; e < 4; ++e) decode4(wds[4 * c4 + e], v + 4 * e);
              tmem_st16(ta + 16 * c4, v);
            }
          } else {
#pragma unroll
            for (int t3 = 0; t3 < 4; ++t3) {
              uint32_t v[16];
              decode3(wds[3 * t3], wds[3 * t3 + 1], wds[3 * t3 + 2], v);
              tmem_st16(ta + 16 * t3, v);
            }
          }
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(B_AFULL(a));
        if (tid == 0 && n / NGRP < 12) tstamp(p, 40 + n / NGRP);

        if (pend) epilogue();
        if (tid == 0 && n / NGRP < 12) tstamp(p, 52 + n / NGRP);
        pend = true;
        pend_n = n;
        pend_piece = w.piece;
        pend_s0 = s0;
        pend_s1 = s1;
        pend_inv = cherry ? 1.f : 1.f / (float)(1 << CE);
        pend_corr = !cherry;
      }
      ++n;
      more = w.next();
    }
    if (tid == 0) tstamp(p, 14);
    if (pend) epilogue();
    for (int pc = tot_piece; pc <= last_piece; ++pc) flush_piece(pc);
    if (tid == (NGRP - 1) * 128) tstamp(p, 15);
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == W_MMA) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------ host side
struct TDeviceInfo { int sms = 0, max_smem = 0; bool ok = false; };
TDeviceInfo tdevice_info(int dev) {
  static TDeviceInfo cache[64];
  if (dev < 0 || dev >= 64) return TDeviceInfo();
  if (!cache[dev].ok) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return TDeviceInfo();
    cache[dev].sms = prop.multiProcessorCount;
    cache[dev].max_smem = (int)prop.sharedMemPerBlockOptin - 1024;
    cache[dev].ok = true;
  }
  return cache[dev];
}

typedef void (*TKernelFn)(const UmmaParams);
template <int NGRP>
TKernelFn tpick(int bits, int sets, int mb) {
  if (bits == 4) {
    if (sets == 1) return mb == 1 ? cq_umma_matvec_kernel<4, 1, 1, NGRP> : cq_umma_matvec_kernel<4, 1, 2, NGRP>;
    return mb == 1 ? cq_umma_matvec_kernel<4, 2, 1, NGRP> : cq_umma_matvec_kernel<4, 2, 2, NGRP>;
  }
  if (sets == 1) return mb == 1 ? cq_umma_matvec_kernel<3, 1, 1, NGRP> : cq_umma_matvec_kernel<3, 1, 2, NGRP>;
  return mb == 1 ? cq_umma_matvec_kernel<3, 2, 1, NGRP> : cq_umma_matvec_kernel<3, 2, 2, NGRP>;
}

int talign_up(int v, int a) { return (v + a - 1) / a * a; }

struct TKnobs { int ngrp, smem_kb, pdl; };
TKnobs tknobs() {
  static TKnobs k = [] {
    TKnobs v{2, 112, 1};
    if (const char* e = getenv("CQ_NGRP")) v.ngrp = atoi(e);
    if (const char* e = getenv("CQ_SMEM_KB")) v.smem_kb = atoi(e);
    if (const char* e = getenv("CQ_PDL")) v.pdl = atoi(e);
    if (v.ngrp != 2 && v.ngrp != 3) v.ngrp = 2;
    return v;
  }();
  return k;
}

}  // namespace

extern "C" int cq_tlayer_matvec(const cq_tlayer* L, const void* x, int ldx, void* y, int ldy, int M, int accumulate,
                                void* scratch, uint32_t* status_word, cq_stream_t stream) {
  if (!L || !L->blob || !x || !y || !scratch) return CQ_ERR_BAD_ARG;
  if (M < 1 || ldx < L->K || ldy < L->N) return CQ_ERR_BAD_ARG;
  int dev = 0;
  CQ_CUDA_TRY(cudaGetDevice(&dev));
  const TDeviceInfo di = tdevice_info(dev);
  if (!di.ok) return CQ_ERR_NO_DEVICE;
  const TKnobs kn = tknobs();
  const __half* xp = (const __half*)x;
  __half* yp = (__half*)y;
  for (int done = 0; done < M; done += 16) {
    const int rows = (M - done) < 16 ? (M - done) : 16;
    const int mb = (rows + 7) / 8;
    UmmaParams p;
    const uint8_t* blob = (const uint8_t*)L->blob;
    p.stream = blob + L->off_stream;
    p.cidx = (const uint16_t*)(blob + L->off_cidx);
    p.osh = (const uint32_t*)(blob + L->off_osh);
    p.x = xp + (size_t)done * ldx;
    p.y = yp + (size_t)done * ldy;
    p.partial = (float*)scratch;
    p.flag = (uint32_t*)((uint8_t*)scratch + (size_t)256 * 2048 * sizeof(float));
    p.status = status_word;
    p.timeline = cq_g_timeline;
    p.M = rows; p.K = L->K; p.N = L->N; p.C = L->C; p.Cp = L->Cp; p.Kp = L->Kp;
    p.n_gran = L->n_gran; p.n_tile = L->n_tile; p.n_cher = L->n_cher;
    p.gran_bytes = L->gran_bytes; p.tile_bytes = L->tile_bytes; p.ipt = L->n_cher + L->n_gran;
    p.ldx = ldx; p.ldy = ldy; p.accumulate = accumulate;
    p.T = (uint32_t)L->n_tile * (uint32_t)p.ipt;
    int grid = di.sms < 256 ? di.sms : 256;
    if ((uint32_t)grid > p.T) grid = (int)p.T;

    p.stage_bytes = talign_up(L->gran_bytes > CQT_CHER_BYTES ? L->gran_bytes : CQT_CHER_BYTES, 128);
    p.sbo16 = mb == 2 ? (WIN_GRAN * 8 * 256) >> 4 : 0;
    p.xwin_bytes = WIN_GRAN * 8 * 256 * mb;
    p.xc_sbo16 = mb == 2 ? (L->n_cher * 256) >> 4 : 0;
    p.nx = 3;
    int off = 0;
    p.off_xwin = off; off = talign_up(off + p.nx * p.xwin_bytes, 128);
    p.off_xc = off;   off = talign_up(off + (L->n_cher ? L->n_cher : 1) * 256 * mb, 128);
    p.off_corr = off; off = talign_up(off + NCORR * L->sets * 16 * 4, 128);
    p.off_cidx = off; off = talign_up(off + (L->Cp + 8) * 2, 128);
    p.off_osh = off;  off = talign_up(off + (L->Kp / 8) * 4, 128);
    p.off_slot = off; off = talign_up(off + 2 * 8 * mb * 128 * 4, 128);
    p.off_pf = off;   off = talign_up(off + 8 * mb * 128 * 4, 128);
    p.off_bar = off;  off = talign_up(off + (2 * MAX_STAGES + 2 * NA + 8 + 2 * NXMAX + 2) * 8, 128);
    p.off_misc = off;
    p.off_ring = off;
    const int fixed = off;
    int budget = kn.smem_kb * 1024;
    if (budget - fixed < 64 * 1024) budget = di.max_smem;
    if (budget > di.max_smem) budget = di.max_smem;
    int stages = (budget - fixed) / p.stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    const uint32_t per = (p.T + grid - 1) / grid;
    if ((uint32_t)stages > per + 1) stages = (int)per + 1;
    if (stages < 2) stages = 2;
    if (fixed + stages * p.stage_bytes > di.max_smem) return CQ_ERR_TOO_LARGE;
    p.stages = stages;
    const int smem = fixed + stages * p.stage_bytes;

    TKernelFn fn = kn.ngrp == 3 ? tpick<3>(L->bits, L->sets, mb) : tpick<2>(L->bits, L->sets, mb);
    CQ_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((kn.ngrp * 4 + 4) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = kn.pdl ? 1 : 0;
    CQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, fn, p));
  }
  return CQ_OK;
}
