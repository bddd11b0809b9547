// Prefill GEMM of a tile-layout CherryQ layer for many activation rows ("tokens"):
//   y[m, n] (+)= sum_k' fp16((u[k', n] - off) * s[group(k'), n]) * x[m, orig(k')]
//              + sum_c  cherry_weight[c, n] * x[m, idx[c]]
// i.e. the reference's dense mode: QuantLinear.unpack() to fp16 followed by F.linear
// (llama/qlinear.py:120-162, 183-195 of the reference project), without ever writing the
// dequantised matrix to memory.  This is the only part of the path that is a dense
// contraction, so it runs on the 5th-generation tensor cores:
//
//   * A operand = weights, 128 rows per CTA tile, dequantised to fp16 by the row's own thread
//     (one thread = one weight row = one TENSOR MEMORY lane) and stored straight into tensor
//     memory with tcgen05.st: exponent-trick unpack (AND-OR into the bits of 1024.0), one exact
//     subtraction and one multiplication by the group scale per fp16 pair, which reproduces
//     unpack()'s fp16 values bit for bit;
//   * B operand = NT tokens of activations per CTA tile (NT = 256, or 128 for calls of at most 128
//     rows), prepared once per call by a small pre-pass kernel (gather into compact column
//     order, canonical K-major UMMA layout) so that the main kernel moves them with plain bulk
//     async copies;
//   * D = 128 rows x NT tokens fp32 in tensor memory, accumulated over the whole K by
//     tcgen05.mma.cta_group::1.kind::f16 (A from TMEM, M = 128, N = NT, K = 16 per instruction);
//     with NT = 128 there are two accumulator buffers, so that the fp16 store of one tile overlaps
//     the MMAs of the next.
//
// Warp roles (704 threads, one CTA per SM, persistent over (token block, row tile) units):
//   warps 0-15  four decode groups (items go round-robin), thread r of a group = row r; a group
//               needs about twice the time the tensor core spends on an item, hence four of them
//   warp 16     MMA issuer (one lane); owns the tensor-memory allocation
//   warp 17     producer (one lane): bulk copies of weight items and activation tiles
//   warps 18-21 epilogue: tcgen05.ld of a finished tile, fp16 store to y
// Every wait is bounded and reports into the status word instead of hanging.
#include <cstdlib>

#include "cq_tile.cuh"

namespace {

constexpr uint32_t WAIT_LIMIT = 1u << 22;
// NT = tokens per tile = UMMA N: 256 (one accumulator buffer; the MMA runs at its full rate) or 128
// (two accumulator buffers; less padding for few tokens).
constexpr int NGRP = 4;                 // decode groups of four warps
constexpr int NA = 4;                   // A slots in tensor memory (64 columns each), one per decode group
constexpr int A_COLS = 64;
constexpr int D_BASE = NA * A_COLS;
constexpr int TMEM_COLS = 512;
constexpr int SW = 4;                   // weight ring stages
constexpr int NTHREADS = (NGRP * 4 + 6) * 32;
// one K = 16 step of the B operand: [token group of 8][k half][8 tokens][16 B] = NT * 32 bytes;
// a granule is 8 steps, a cherry item one
__host__ __device__ constexpr int b_kstep_bytes(int nt) { return nt * 32; }
__host__ __device__ constexpr int b_gran_bytes(int nt) { return nt * 256; }

struct PrefillParams {
  const uint8_t* stream;     // tile-layout weight stream
  const uint8_t* xb;         // staged activations: [token block][cherry items][granules]
  __half* y;
  uint32_t* status;
  int M, N, n_gran, n_tile, n_cher, gran_bytes, tile_bytes, ldy, accumulate;
  uint32_t n_units;          // token blocks x row tiles
  unsigned long long xb_blk_bytes;
  int wstage_bytes, sb, off_wring, off_bring, off_bar;   // sb = activation ring stages
  int split;                 // parts the items of a unit are divided into (split-K), 1 = none
  float* partial;            // [unit][part][row tile][128 rows][NT] fp32 partial tiles (split > 1)
  uint32_t* arrived;         // [unit] parts finished so far (split > 1)
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
// Bounded wait: gives up after WAIT_LIMIT polls (at once when the CTA already gave up), records
// which wait failed in the status word and lets the caller run on to the common exit.
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
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem_d] (+)= A[tmem_a] * B[desc_b]: fp16 inputs, fp32 accumulate, shape from the instruction descriptor
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
__device__ __forceinline__ void tmem_ld16(uint32_t addr, float* v) {
  uint32_t r[16];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(addr) : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major, unswizzled operand: rows of a core matrix 16 B
// apart, the two 8-column halves of a 16-column step `lbo` bytes apart, 8-row groups `sbo` apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo16, uint32_t sbo16) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)lbo16 << 16) | ((uint64_t)sbo16 << 32) | ((uint64_t)1 << 46);
}

// ------------------------------------------------------------------ dequantisation to fp16
// A code field at mantissa bit p OR-ed into the bits of fp16 1024.0 is the number 1024 + 2^p u.
// Subtracting 1024 + 2^p off is exact (the result is 2^p (u - off), a small multiple of 2^(p-1)),
// and the product with s * 2^-p is (u - off) * s rounded once to fp16: exactly the value
// unpack() computes as fp16(q + 0.5) * s (llama/qlinear.py:139-146 of the reference project).
constexpr uint32_t MAGIC = 0x64006400u;
__device__ __forceinline__ uint32_t dup16(uint32_t h) { return h | (h << 16); }
// fp16 bits of 1024 + 2^p * off
template <int BITS> __device__ __forceinline__ constexpr uint32_t center(int pbit) {
  return BITS == 4 ? (pbit == 2 ? 0x641Eu : 0x65E0u)                       // 1054, 1504
                   : (pbit == 1 ? 0x6407u : (pbit == 4 ? 0x6438u : 0x65C0u));   // 1031, 1080, 1472
}
__device__ __forceinline__ uint32_t pow2_neg(int pbit) { return (uint32_t)(15 - pbit) << 10; }   // fp16 bits of 2^-p

// One 4-bit word (8 codes) -> 4 fp16 pairs; sc2 / sc6 = (s * 2^-2, s * 2^-2), (s * 2^-6, s * 2^-6)
__device__ __forceinline__ void dequant4(uint32_t w, uint32_t sc2, uint32_t sc6, uint32_t* out) {
  const uint32_t v1 = w << 2, v2 = w >> 6;
  const uint32_t c2 = dup16(center<4>(2)), c6 = dup16(center<4>(6));
  out[0] = hmul2_u32(hsub2_u32((v1 & 0x003C003Cu) | MAGIC, c2), sc2);
  out[1] = hmul2_u32(hsub2_u32((v1 & 0x03C003C0u) | MAGIC, c6), sc6);
  out[2] = hmul2_u32(hsub2_u32((v2 & 0x003C003Cu) | MAGIC, c2), sc2);
  out[3] = hmul2_u32(hsub2_u32((v2 & 0x03C003C0u) | MAGIC, c6), sc6);
}
// Three 3-bit words (32 codes) -> 16 fp16 pairs; sc1 / sc4 / sc7 = s * 2^-1, 2^-4, 2^-7 pairs
__device__ __forceinline__ void dequant3(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t sc1, uint32_t sc4, uint32_t sc7,
                                         uint32_t* out) {
  const uint32_t c1 = dup16(center<3>(1)), c4 = dup16(center<3>(4)), c7 = dup16(center<3>(7));
  const uint32_t w[3] = {w0, w1, w2};
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const uint32_t v = w[i] >> 6;
    out[5 * i + 0] = hmul2_u32(hsub2_u32((w[i] & 0x000E000Eu) | MAGIC, c1), sc1);   // field at bit 1
    out[5 * i + 1] = hmul2_u32(hsub2_u32((w[i] & 0x00700070u) | MAGIC, c4), sc4);   // bit 4
    out[5 * i + 2] = hmul2_u32(hsub2_u32((w[i] & 0x03800380u) | MAGIC, c7), sc7);   // bit 7
    out[5 * i + 3] = hmul2_u32(hsub2_u32((v & 0x00700070u) | MAGIC, c4), sc4);      // bit 10 -> 4
    out[5 * i + 4] = hmul2_u32(hsub2_u32((v & 0x03800380u) | MAGIC, c7), sc7);      // bit 13 -> 7
  }
  uint32_t r = ((w0 << 7) & 0x00800080u) | MAGIC;     // pair 15: one bit from each word, at bits 7..9
  r |= (w1 << 8) & 0x01000100u;
  r |= (w2 << 9) & 0x02000200u;
  out[15] = hmul2_u32(hsub2_u32(r, c7), sc7);
}

// ------------------------------------------------------------------ activation pre-pass
// xb[token block][item][...] in the layout the MMA reads from shared memory: per K = 16 step
// [token group of 8][k half][token in group][8 fp16]; cherry items (16 cherry columns) first, then
// the granules (128 compact columns = 8 steps).  Tokens past M are not written.
__global__ void prefill_stage_x_kernel(const __half* __restrict__ x, int ldx, int M, const uint32_t* __restrict__ osh,
                                       const uint16_t* __restrict__ cidx, int C, int Kc, int n_gran, int n_cher,
                                       uint8_t* __restrict__ xb, unsigned long long blk_bytes, int n_mblk, int NT) {
  const int per_tok = 2 * n_cher + 16 * n_gran;            // octets per token
  // Only real tokens are staged: the padding columns of the last token block feed accumulator
  // columns that are never read back (each output column depends on its own token only).
  const long long total = (long long)M * per_tok;
  (void)n_mblk;
  const int B_KSTEP_BYTES = b_kstep_bytes(NT), B_GRAN_BYTES = b_gran_bytes(NT), B_CHER_BYTES = B_KSTEP_BYTES;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(id / per_tok), oi = (int)(id % per_tok);
    const int mb = m / NT, ml = m % NT;
    unsigned short h[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) h[e] = 0;
    uint8_t* dst;
    const unsigned short* xr = reinterpret_cast<const unsigned short*>(x) + (size_t)m * ldx;
    if (oi < 2 * n_cher) {
      const int j = oi >> 1, hh = oi & 1;
      if (m < M) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int c = 16 * j + 8 * hh + e;
          if (c < C) h[e] = __ldg(xr + cidx[c]);
        }
      }
      dst = xb + (size_t)mb * blk_bytes + (size_t)j * B_CHER_BYTES + (ml >> 3) * 256 + hh * 128 + (ml & 7) * 16;
    } else {
      const int o = oi - 2 * n_cher, g = o >> 4, oo = o & 15;
      const int k0 = 8 * o;
      const uint32_t sh = osh[o];
      if (m < M && sh != 0xFFFFFFFFu) {
        const int lo0 = (int)(sh & 0xFFFFu), lo7 = (int)(sh >> 16);
        if (lo0 == lo7 && ((k0 + lo0) & 1) == 0 && (((uintptr_t)xr) & 3) == 0) {
          // eight consecutive columns at a 4-byte aligned address (K' is a multiple of 8: all exist)
          const uint32_t* s32 = reinterpret_cast<const uint32_t*>(xr + k0 + lo0);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t w = __ldg(s32 + i);
            h[2 * i] = (unsigned short)(w & 0xFFFFu);
            h[2 * i + 1] = (unsigned short)(w >> 16);
          }
        } else {
          int sft = lo0;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            // cherry columns inside the octet: the shift grows from lo0 to lo7 along it
            while (sft < lo7 && (int)cidx[sft] - sft <= k0 + e) ++sft;
            if (k0 + e < Kc) h[e] = __ldg(xr + k0 + e + sft);
          }
        }
      }
      dst = xb + (size_t)mb * blk_bytes + (size_t)n_cher * B_CHER_BYTES + (size_t)g * B_GRAN_BYTES +
            (oo >> 1) * B_KSTEP_BYTES + (ml >> 3) * 256 + (oo & 1) * 128 + (ml & 7) * 16;
    }
    uint4 v;
    v.x = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
    v.y = (uint32_t)h[2] | ((uint32_t)h[3] << 16);
    v.z = (uint32_t)h[4] | ((uint32_t)h[5] << 16);
    v.w = (uint32_t)h[6] | ((uint32_t)h[7] << 16);
    *reinterpret_cast<uint4*>(dst) = v;
  }
}

// ------------------------------------------------------------------ main kernel
// RT = row tiles of 128 rows per unit: with two, one staged activation tile feeds two weight tiles,
// which halves the activation bytes an SM has to pull from L2 per flop.
template <int BITS, int SETS, int NT, int RT>
__global__ void __launch_bounds__(NTHREADS, 1) cq_prefill_kernel(const PrefillParams p) {
  constexpr int W_MMA = NGRP * 4, W_PROD = NGRP * 4 + 1;
  constexpr int ND = (NT * RT == 128) ? 2 : 1;            // accumulator buffers (RT * NT columns each)
  constexpr int SBMAX = 4;
  constexpr int B_KSTEP_BYTES = b_kstep_bytes(NT), B_GRAN_BYTES = b_gran_bytes(NT), B_CHER_BYTES = B_KSTEP_BYTES;
  // instruction descriptor: fp32 accumulate, fp16 A and B, both K-major, N = NT, M = 128
  constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | (8u << 24);
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_abort;
  __shared__ uint32_t s_tmem;
  __shared__ int s_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t grid = gridDim.x, cta = blockIdx.x;
  const uint32_t NCH = (uint32_t)p.n_cher, IPT = NCH + (uint32_t)p.n_gran;
  const uint32_t NTILE = (uint32_t)p.n_tile;
  const uint32_t NPAIR = (NTILE + RT - 1) / RT;          // units per token block
  const uint32_t SB = (uint32_t)p.sb;
  const uint32_t SPLIT = (uint32_t)p.split;
  const uint32_t n_work = p.n_units * SPLIT;               // work items: (unit, part), part fastest

  const uint32_t bar0 = smem_u32(smem + p.off_bar);
  auto B_WFULL = [&](uint32_t s) { return bar0 + 8 * s; };
  auto B_WEMPTY = [&](uint32_t s) { return bar0 + 8 * (SW + s); };
  auto B_BFULL = [&](uint32_t s) { return bar0 + 8 * (2 * SW + s); };
  auto B_BEMPTY = [&](uint32_t s) { return bar0 + 8 * (2 * SW + SBMAX + s); };
  auto B_AFULL = [&](uint32_t a) { return bar0 + 8 * (2 * SW + 2 * SBMAX + a); };
  auto B_AEMPTY = [&](uint32_t a) { return bar0 + 8 * (2 * SW + 2 * SBMAX + NA + a); };
  auto B_DFULL = [&](uint32_t d) { return bar0 + 8 * (2 * SW + 2 * SBMAX + 2 * NA + d); };
  auto B_DEMPTY = [&](uint32_t d) { return bar0 + 8 * (2 * SW + 2 * SBMAX + 2 * NA + 2 + d); };

  if (tid == 0) {
    s_abort = 0;
    for (uint32_t s = 0; s < SW; ++s) { mbar_init(B_WFULL(s), 1); mbar_init(B_WEMPTY(s), 4); }
    for (uint32_t s = 0; s < SB; ++s) { mbar_init(B_BFULL(s), 1); mbar_init(B_BEMPTY(s), 1); }
    for (uint32_t a = 0; a < NA; ++a) { mbar_init(B_AFULL(a), 4); mbar_init(B_AEMPTY(a), 1); }
    for (uint32_t d = 0; d < ND; ++d) { mbar_init(B_DFULL(d), 1); mbar_init(B_DEMPTY(d), 4); }
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
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == W_PROD) {
    // ================================================================ producer
    if (lane == 0) {
      // the staged activations are written by the kernel launched just before this one
      asm volatile("griddepcontrol.wait;" ::: "memory");
      const uint32_t wring = smem_u32(smem + p.off_wring), bring = smem_u32(smem + p.off_bring);
      uint32_t n = 0, nb = 0;      // weight items and activation tiles issued so far
      for (uint32_t wk = cta; wk < n_work; wk += grid) {
        const uint32_t u = wk / SPLIT, part = wk - u * SPLIT;
        const uint32_t j0 = part * IPT / SPLIT, j1 = (part + 1) * IPT / SPLIT;
        const uint32_t mb = u / NPAIR, t0 = (u - mb * NPAIR) * RT;
        const uint32_t ntr = min((uint32_t)RT, NTILE - t0);
        // offsets of item j0 inside a row tile's block and inside the token block's staged activations
        const uint32_t c0 = min(j0, NCH), g0 = j0 - c0;
        size_t woff = (size_t)c0 * CQT_CHER_BYTES + (size_t)g0 * p.gran_bytes;
        const uint8_t* bsrc = p.xb + (size_t)mb * p.xb_blk_bytes + (size_t)c0 * B_CHER_BYTES + (size_t)g0 * B_GRAN_BYTES;
        for (uint32_t j = j0; j < j1; ++j, ++nb) {
          const bool cherry = j < NCH;
          const uint32_t sb = nb % SB;
          const uint32_t wbytes = cherry ? (uint32_t)CQT_CHER_BYTES : (uint32_t)p.gran_bytes;
          const uint32_t bbytes = cherry ? (uint32_t)B_CHER_BYTES : (uint32_t)B_GRAN_BYTES;
          for (uint32_t rt = 0; rt < ntr; ++rt, ++n) {
            const uint32_t sw = n % SW;
            if (n >= SW) mbar_wait(B_WEMPTY(sw), ((n / SW) - 1) & 1, &s_abort, p.status, 1u);
            mbar_expect_tx(B_WFULL(sw), wbytes);
            bulk_g2s(wring + sw * (uint32_t)p.wstage_bytes, p.stream + (size_t)(t0 + rt) * p.tile_bytes + woff, wbytes,
                     B_WFULL(sw));
          }
          if (nb >= SB) mbar_wait(B_BEMPTY(sb), ((nb / SB) - 1) & 1, &s_abort, p.status, 2u);
          mbar_expect_tx(B_BFULL(sb), bbytes);
          bulk_g2s(bring + sb * (uint32_t)B_GRAN_BYTES, bsrc, bbytes, B_BFULL(sb));
          woff += wbytes;
          bsrc += bbytes;
        }
      }
    }
  } else if (warp == W_MMA) {
    // ================================================================ MMA issuer
    if (lane == 0) {
      const uint32_t bring = smem_u32(smem + p.off_bring);
      uint32_t n = 0, nb = 0, lu = 0;
      for (uint32_t wk = cta; wk < n_work; wk += grid, ++lu) {
        const uint32_t u = wk / SPLIT, part = wk - u * SPLIT;
        const uint32_t j0 = part * IPT / SPLIT, j1 = (part + 1) * IPT / SPLIT;
        const uint32_t mb = u / NPAIR, t0 = (u - mb * NPAIR) * RT;
        const uint32_t ntr = min((uint32_t)RT, NTILE - t0);
        const uint32_t dbuf = lu % ND;
        if (lu >= ND) mbar_wait(B_DEMPTY(dbuf), ((lu / ND) - 1) & 1, &s_abort, p.status, 4u);
        for (uint32_t j = j0; j < j1; ++j, ++nb) {
          const uint32_t sb = nb % SB;
          mbar_wait(B_BFULL(sb), (nb / SB) & 1, &s_abort, p.status, 16u);
          const uint32_t bbase = bring + sb * (uint32_t)B_GRAN_BYTES;
          for (uint32_t rt = 0; rt < ntr; ++rt, ++n) {
            const uint32_t a = n % NA;
            const uint32_t td = tmem + D_BASE + (dbuf * RT + rt) * NT;
            mbar_wait(B_AFULL(a), (n / NA) & 1, &s_abort, p.status, 8u);
            tc_fence_after();
            const uint32_t ta = tmem + a * A_COLS;
            if (j < NCH) {
              umma_ts(td, ta, smem_desc(bbase, 8, 16), IDESC, j != j0);
            } else {
#pragma unroll
              for (uint32_t ks = 0; ks < 8; ++ks)
                umma_ts(td, ta + ks * 8, smem_desc(bbase + ks * B_KSTEP_BYTES, 8, 16), IDESC, (j != j0 || ks != 0));
            }
            tc_commit(B_AEMPTY(a));
          }
          tc_commit(B_BEMPTY(sb));
        }
        tc_commit(B_DFULL(dbuf));
      }
    }
  } else if (warp < W_MMA) {
    // ================================================================ decode groups
    const int grp = warp >> 2;
    const int row = (warp & 3) * 32 + lane;                 // row of the tile = tensor-memory lane
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint8_t* wring = smem + p.off_wring;
    uint32_t n = 0;
    for (uint32_t wk = cta; wk < n_work; wk += grid) {
      const uint32_t u = wk / SPLIT, part = wk - u * SPLIT;
      const uint32_t j0 = part * IPT / SPLIT, j1 = (part + 1) * IPT / SPLIT;
      const uint32_t mbu = u / NPAIR, t0 = (u - mbu * NPAIR) * RT;
      const uint32_t ntr = min((uint32_t)RT, NTILE - t0);
      for (uint32_t jj = 0; jj < (j1 - j0) * ntr; ++jj, ++n) {
        const uint32_t j = j0 + jj / ntr;          // items of the work item: (item j, row tile 0), (j, 1), ...
        if ((int)(n % NGRP) != grp) continue;
        const uint32_t sw = n % SW, a = n % NA;
        mbar_wait(B_WFULL(sw), (n / SW) & 1, &s_abort, p.status, 32u);
        const uint8_t* item = wring + (size_t)sw * p.wstage_bytes;
        const bool cherry = j < NCH;
        uint4 raw[BITS];
        uint32_t s0 = 0, s1 = 0;
        if (cherry) {
          raw[0] = *reinterpret_cast<const uint4*>(item + row * 16);
          raw[1] = *reinterpret_cast<const uint4*>(item + 2048 + row * 16);
        } else {
#pragma unroll
          for (int q = 0; q < BITS; ++q) raw[q] = *reinterpret_cast<const uint4*>(item + q * 2048 + row * 16);
          const unsigned short* sc = reinterpret_cast<const unsigned short*>(item + 2048 * BITS);
          s0 = dup16(sc[row]);
          s1 = (SETS == 2) ? dup16(sc[128 + row]) : s0;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(B_WEMPTY(sw));
        if (n >= NA) mbar_wait(B_AEMPTY(a), ((n / NA) - 1) & 1, &s_abort, p.status, 64u);
        tc_fence_after();
        const uint32_t ta = tmem + lane_addr + a * A_COLS;
        if (cherry) {
          const uint32_t v[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
          tmem_st8(ta, v);
        } else {
          const uint32_t* wds = reinterpret_cast<const uint32_t*>(raw);
          if constexpr (BITS == 4) {
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              const uint32_t s = (c4 < 2) ? s0 : s1;
              const uint32_t sc2 = hmul2_u32(s, dup16(pow2_neg(2))), sc6 = hmul2_u32(s, dup16(pow2_neg(6)));
              uint32_t v[16];
#pragma unroll
              for (int e = 0; e < 4; ++e) dequant4(wds[4 * c4 + e], sc2, sc6, v + 4 * e);
              tmem_st16(ta + 16 * c4, v);
            }
          } else {
#pragma unroll
            for (int t3 = 0; t3 < 4; ++t3) {
              const uint32_t s = (t3 < 2) ? s0 : s1;
              const uint32_t sc1 = hmul2_u32(s, dup16(pow2_neg(1))), sc4 = hmul2_u32(s, dup16(pow2_neg(4))),
                             sc7 = hmul2_u32(s, dup16(pow2_neg(7)));
              uint32_t v[16];
              dequant3(wds[3 * t3], wds[3 * t3 + 1], wds[3 * t3 + 2], sc1, sc4, sc7, v);
              tmem_st16(ta + 16 * t3, v);
            }
          }
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(B_AFULL(a));
      }
    }
  } else {
    // ================================================================ epilogue (last four warps)
    const int quad = warp & 3;                              // the tensor-memory lanes this warp may read
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int etid = tid - (NGRP * 4 + 2) * 32;             // 0..127 among the epilogue threads
    uint32_t lu = 0;
    for (uint32_t wk = cta; wk < n_work; wk += grid, ++lu) {
      const uint32_t u = wk / SPLIT, part = wk - u * SPLIT;
      const uint32_t mb = u / NPAIR, t0 = (u - mb * NPAIR) * RT;
      const uint32_t ntr = min((uint32_t)RT, NTILE - t0);
      const uint32_t dbuf = lu % ND;
      mbar_wait(B_DFULL(dbuf), (lu / ND) & 1, &s_abort, p.status, 128u);
      tc_fence_after();
      const int tok0 = (int)mb * NT;
      // 16-token chunks of this block that hold real tokens (the rest of the tile is padding)
      const int n_chunks = min(NT / 16, (p.M - tok0 + 15) / 16);
      auto store_row = [&](const float (&v)[16], int n_row, int c) {
        if (n_row < p.N) {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int tok = tok0 + c * 16 + e;
            if (tok < p.M) {
              __half* yp = p.y + (size_t)tok * p.ldy + n_row;
              float val = v[e];
              if (p.accumulate) val += __half2float(*yp);
              *yp = __float2half(val);
            }
          }
        }
      };
      if (SPLIT == 1) {
        for (uint32_t rt = 0; rt < ntr; ++rt) {
          const int n_row = (int)(t0 + rt) * 128 + row;
#pragma unroll 1
          for (int c = 0; c < n_chunks; ++c) {
            float v[16];
            tmem_ld16(tmem + lane_addr + D_BASE + (dbuf * RT + rt) * NT + c * 16, v);
            tmem_wait_ld();
            store_row(v, n_row, c);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(B_DEMPTY(dbuf));
      } else {
        // split-K: park this part's fp32 tile; the part that arrives last adds the parts in a fixed
        // order (deterministic sums) and stores the outputs
        float* mine = p.partial + ((size_t)(u * SPLIT + part) * RT) * 128 * NT;
        for (uint32_t rt = 0; rt < ntr; ++rt) {
#pragma unroll 1
          for (int c = 0; c < n_chunks; ++c) {
            float v[16];
            tmem_ld16(tmem + lane_addr + D_BASE + (dbuf * RT + rt) * NT + c * 16, v);
            tmem_wait_ld();
            float4* dst = reinterpret_cast<float4*>(mine + ((size_t)rt * 128 + row) * NT + c * 16);
#pragma unroll
            for (int e = 0; e < 4; ++e) dst[e] = make_float4(v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(B_DEMPTY(dbuf));
        __threadfence();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (etid == 0) s_last = (atomicAdd(p.arrived + u, 1u) == SPLIT - 1) ? 1 : 0;
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (s_last) {
          __threadfence();
          const float* base = p.partial + ((size_t)(u * SPLIT) * RT) * 128 * NT;
          for (uint32_t rt = 0; rt < ntr; ++rt) {
            const int n_row = (int)(t0 + rt) * 128 + row;
#pragma unroll 1
            for (int c = 0; c < n_chunks; ++c) {
              float v[16];
#pragma unroll
              for (int e = 0; e < 16; ++e) v[e] = 0.f;
              for (uint32_t q = 0; q < SPLIT; ++q) {
                const float4* src = reinterpret_cast<const float4*>(base + (((size_t)q * RT + rt) * 128 + row) * NT + c * 16);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float4 f = __ldcg(src + e);
                  v[4 * e] += f.x; v[4 * e + 1] += f.y; v[4 * e + 2] += f.z; v[4 * e + 3] += f.w;
                }
              }
              store_row(v, n_row, c);
            }
          }
          if (etid == 0) p.arrived[u] = 0u;          // ready for the next call
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == W_MMA) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

struct PDeviceInfo { int sms = 0, max_smem = 0; bool ok = false; };
PDeviceInfo pdevice_info(int dev) {
  static PDeviceInfo cache[64];
  if (dev < 0 || dev >= 64) return PDeviceInfo();
  if (!cache[dev].ok) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return PDeviceInfo();
    cache[dev].sms = prop.multiProcessorCount;
    cache[dev].max_smem = (int)prop.sharedMemPerBlockOptin - 1024;
    cache[dev].ok = true;
  }
  return cache[dev];
}

int palign_up(int v, int a) { return (v + a - 1) / a * a; }

typedef void (*PKernelFn)(const PrefillParams);
template <int NT, int RT>
PKernelFn ppick(int bits, int sets) {
  if (bits == 4) return sets == 1 ? cq_prefill_kernel<4, 1, NT, RT> : cq_prefill_kernel<4, 2, NT, RT>;
  return sets == 1 ? cq_prefill_kernel<3, 1, NT, RT> : cq_prefill_kernel<3, 2, NT, RT>;
}

// Tile shape for a call of M rows: 0 = 128 rows x 128 tokens (two accumulator buffers), 1 = 128 x 256,
// 2 = 256 x 128.
int tile_shape(int M, int n_tile) {
  (void)n_tile;
  // measured on 4096 -> 11008, 2048 tokens: 128 x 256 tiles 938 TFLOP/s, 128 x 128 673, 256 x 128 613: the
  // tensor-memory MMA only reaches its rate at N = 256
  return M > 128 ? 1 : 0;
}

unsigned long long xb_block_bytes(const cq_tlayer* L, int nt) {
  return (unsigned long long)L->n_cher * b_kstep_bytes(nt) + (unsigned long long)L->n_gran * b_gran_bytes(nt);
}

// Split-K for calls whose units do not fill the SMs (few tokens): into how many parts the items of
// a unit are divided so that the parts fill the SMs about evenly.
constexpr int MAX_SPLIT = 4;
int pick_split(int n_units, int items, int sms) {
  int best = 1;
  if (n_units < sms) {
    double best_t = 1.0;                                   // makespan, in whole units
    for (int sp = 2; sp <= MAX_SPLIT; ++sp) {
      const int waves = (n_units * sp + sms - 1) / sms;
      const double t = (double)waves / sp + 0.04 * sp;     // + a small cost per part for the reduction
      if (t < best_t - 1e-9) { best_t = t; best = sp; }
    }
  }
  if (best > items) best = items;
  return best < 1 ? 1 : best;
}

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// Workspace: staged activations | fp32 partial tiles of split-K | arrival counters (one per unit).
size_t xb_bytes_for(const cq_tlayer* L, int M) {
  // (both tile widths stage the same bytes per token; round up to the wider one)
  const size_t n_mblk = ((size_t)M + 255) / 256;
  return align256(n_mblk * (size_t)xb_block_bytes(L, 256));
}
// Split-K only happens while the units do not fill the SMs: at most 255 units of MAX_SPLIT parts.
size_t partial_bytes_for(const cq_tlayer* L, int M) {
  const int nt = M > 128 ? 256 : 128;
  const size_t units = (((size_t)M + nt - 1) / nt) * (size_t)L->n_tile;
  return units < 256 ? align256(units * MAX_SPLIT * 128 * nt * sizeof(float)) : 0;
}
constexpr size_t COUNTER_BYTES = 256 * sizeof(uint32_t);

}  // namespace

extern "C" size_t cq_tlayer_gemm_workspace_bytes(const cq_tlayer* L, int M) {
  if (!L || M < 1) return 0;
  return xb_bytes_for(L, M) + partial_bytes_for(L, M) + COUNTER_BYTES;
}

extern "C" int cq_tlayer_gemm(const cq_tlayer* L, const void* x, int ldx, void* y, int ldy, int M, int accumulate,
                              void* workspace, uint32_t* status_word, cq_stream_t stream) {
  if (!L || !L->blob || !x || !y || !workspace) return CQ_ERR_BAD_ARG;
  if (M < 1 || ldx < L->K || ldy < L->N) return CQ_ERR_BAD_ARG;
  if (((uintptr_t)x & 1) || ((uintptr_t)y & 1) || ((uintptr_t)workspace & 127)) return CQ_ERR_BAD_ARG;
  int dev = 0;
  CQ_CUDA_TRY(cudaGetDevice(&dev));
  const PDeviceInfo di = pdevice_info(dev);
  if (!di.ok) return CQ_ERR_NO_DEVICE;
  cudaStream_t st = (cudaStream_t)stream;
  const uint8_t* blob = (const uint8_t*)L->blob;
  const int shape = tile_shape(M, L->n_tile);
  const int NT = shape == 1 ? 256 : 128, RT = shape == 2 ? 2 : 1;
  const int n_mblk = (M + NT - 1) / NT;
  const unsigned long long blk = xb_block_bytes(L, NT);

  {
    const long long total = (long long)M * (2 * L->n_cher + 16 * L->n_gran);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    prefill_stage_x_kernel<<<(int)blocks, 256, 0, st>>>(
        (const __half*)x, ldx, M, (const uint32_t*)(blob + L->off_osh), (const uint16_t*)(blob + L->off_cidx), L->C,
        L->Kc, L->n_gran, L->n_cher, (uint8_t*)workspace, blk, n_mblk, NT);
    CQ_CUDA_TRY(cudaGetLastError());
  }

  PrefillParams p;
  p.stream = blob + L->off_stream;
  p.xb = (const uint8_t*)workspace;
  p.y = (__half*)y;
  p.status = status_word;
  p.M = M; p.N = L->N; p.n_gran = L->n_gran; p.n_tile = L->n_tile; p.n_cher = L->n_cher;
  p.gran_bytes = L->gran_bytes; p.tile_bytes = L->tile_bytes; p.ldy = ldy; p.accumulate = accumulate;
  p.n_units = (uint32_t)n_mblk * (uint32_t)((L->n_tile + RT - 1) / RT);
  // Split-K pays for decode-sized batches only: the reduction costs about 4 us per 16-token chunk
  // (measured: 128 tokens through 4096 -> 11008 take 61 us in three parts against 37 us unsplit, 16
  // tokens through 4096 -> 4096 21 us in four parts against 35 us).
  p.split = (M <= 32 && p.n_units < 256 && partial_bytes_for(L, M) > 0 && RT == 1)
                ? pick_split((int)p.n_units, L->n_cher + L->n_gran, di.sms) : 1;
  p.partial = (float*)((uint8_t*)workspace + xb_bytes_for(L, M));
  p.arrived = (uint32_t*)((uint8_t*)workspace + xb_bytes_for(L, M) + partial_bytes_for(L, M));
  if (p.split > 1) CQ_CUDA_TRY(cudaMemsetAsync(p.arrived, 0, COUNTER_BYTES, st));
  p.xb_blk_bytes = blk;
  p.wstage_bytes = palign_up(L->gran_bytes > CQT_CHER_BYTES ? L->gran_bytes : CQT_CHER_BYTES, 128);
  int off = 0;
  p.off_bar = off;   off = palign_up(off + (2 * SW + 2 * 4 + 2 * NA + 4) * 8, 128);
  p.off_wring = off; off = palign_up(off + SW * p.wstage_bytes, 128);
  p.off_bring = off;
  p.sb = (di.max_smem - off) / b_gran_bytes(NT);
  if (p.sb > 4) p.sb = 4;
  if (p.sb < 2) return CQ_ERR_TOO_LARGE;
  const int smem = off + p.sb * b_gran_bytes(NT);
  int grid = di.sms;
  if ((uint32_t)grid > p.n_units * (uint32_t)p.split) grid = (int)(p.n_units * (uint32_t)p.split);

  PKernelFn fn = shape == 1 ? ppick<256, 1>(L->bits, L->sets)
                            : (shape == 2 ? ppick<128, 2>(L->bits, L->sets) : ppick<128, 1>(L->bits, L->sets));
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
  return CQ_OK;
}
