// Decode matvec for ONE activation row: y (1, N) fp16 = [y +] x (1, K) fp16 . W^T.
//
// Replaces the reference's batch-1 use of VecQuant4MatMulKernelCherryQBatchedHalf and
// VecQuant3MatMulKernelCherryQBatched(G64)Half (csrc/quant_cuda_kernel.cu:718-835, 558-672,
// 316-438 of the reference project): one thread per output column there, byte loads at stride N,
// fp16 atomics.
//
// What bounds a batch-1 matvec in a chain of dependent launches is not only the bytes: every CTA
// has to wait for the previous kernel (about 1.3 us after its last CTA left), and everything that
// needs x is serial after that wait.  The kernel is built around making that serial part short:
//
//   * layout (cq_rlayer, include/cherryq.h): tiles of 16 output rows, one contiguous record per
//     tile; a CTA owns consecutive tiles, i.e. one contiguous byte range.  It asks for that range
//     with bulk async copies (cp.async.bulk + mbarrier transaction counts) into shared memory the
//     moment it starts, BEFORE the dependency wait: weights are constants, only x is not.  HBM
//     streams while the CTA waits and stages.  A ring of tile slots serves layers whose share
//     exceeds shared memory;
//   * K is split over the warps of the CTA: warp w owns a few 128-column groups of EVERY tile.
//     So a warp needs only its own slice of x: it loads that slice itself (coalesced, no
//     CTA-wide barrier), quantises it to two signed-byte planes (q = 128 hi + lo, |q| <= 16256,
//     one step size per group) and keeps the result as B fragments of the integer tensor-core
//     instruction mma.sync.m16n8k32 (u8 x s8 -> s32) in registers for the whole kernel;
//   * per tile and group a lane reads 32 (4-bit) / 24 (3-bit) bytes, masks them into A fragments
//     (one logic operation per four codes; the high nibbles stay where they are, as 16 u) and
//     issues four MMAs; columns 0 / 1 of B carry the hi / lo plane, so the sums are exact:
//         sum_k (u_k - off) x_k = sx (128 sum u hi + sum u lo) - off sx sum q;
//     cherry columns are one fp16 mma.sync.m16n8k16 per tile;
//   * the warps' partial sums of a tile meet in shared memory and are added in a fixed order:
//     no atomics, no scratch, no cross-CTA traffic, bit-identical runs.
#include <map>
#include <mutex>
#include <utility>

#include "cq_common.cuh"
#include "cq_peer.cuh"

namespace {

constexpr uint32_t RV_WAIT_LIMIT = 1u << 22;
constexpr int RV_MAX_SLOTS = 16;            // ring slots (tiles resident in shared memory at a time)

constexpr int RV_MAX_SEG = 4;               // layers one launch can serve (they share the activations)
constexpr int RV_MAX_ROWS = 4;              // activation rows one launch can serve (two MMA columns each)
constexpr int RV_MAX_KSPLIT = 8;            // CTAs that can share a tile, each taking a part of the columns

// One layer of a launch: a range of CTAs works on it.
struct RowvecSeg {
  const uint8_t* tiles;     // tile records: [NG groups][scales][cherry blocks]
  const uint16_t* perm;     // [NG * 128] original column of each compact column, K for padding
  const uint16_t* cidx;     // [Cp] sorted cherry columns
  __half* y;
  float* work;              // [ks][NT][M][16] partial sums of the column parts (layers split along K only)
  unsigned int* counters;   // [NT] arrivals per unit, indexed by the unit's first tile; zero between launches
  int N, NT;
  int cta0;                 // first CTA of the range
  int tiles_q, tiles_r;     // unit u of the range (ks consecutive CTAs) owns tiles_q (+1 if u < tiles_r) consecutive tiles
};

struct RowvecParams {
  RowvecSeg seg[RV_MAX_SEG];
  int nseg;
  const __half* x;
  const __half* x2;         // not null: the activations are silu(x) * x2, element by element (the SwiGLU of a gated MLP
                            // computed while the down projection stages its input); same shape and stride as x
  int M, ldx, ldy;          // activation rows of the call (1..4) and the row strides of x and y, in elements
  uint32_t* status;         // may be null
  int K, C, NG, ncb;        // common to the layers of a launch; ncb = cherry blocks of 16 columns
  int tile_bytes, scal_off, cher_off;        // a tile record in global memory
  // Layers of more than 64 groups are split along K: ks consecutive CTAs (a unit) share their tiles, CTA j of a
  // unit takes groups [j NGp, (j + 1) NGp) (and the cherry columns if j == 0) and keeps only that part of a
  // tile in its ring slot; the unit's CTA that finishes last adds the parts' sums in part order.
  int ks, NGp;
  int grp_bytes, set_bytes;                  // 256 * bits; sets * 32 (scales of one group)
  int slot_bytes, scal_off_s, cher_off_s;    // a ring slot: [groups of the part][their scales][cherry blocks]
  int slots;                // ring slots in use
  int inflight;             // tiles the copy warp keeps outstanding
  int slice_halves;         // halves of a warp's raw activation slice in shared memory
  int off_slice, off_part, off_bar, off_tiles;   // shared-memory sections (bytes)
  int accumulate;
  // Column-parallel deployments: with gather != 0 the CTA of the grid that finishes last runs the
  // exchange of the ranks' output slices over peer memory (cq_peer.cuh) before the kernel ends, so the
  // gathered rows are complete when the next kernel of the stream starts.  One layer per launch.
  int gather;
  cq_peer::PeerGatherParams peer;
};

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t rv_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void rv_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void rv_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void rv_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// silu(g) * u as the decode harness computes it in two kernels' worth of roundings: the activation is an
// fp16 tensor, the product an fp16 multiplication
__device__ __forceinline__ __half rv_swiglu(__half g, __half u) {
  const float gf = __half2float(g);
  return __hmul(__float2half(gf / (1.f + __expf(-gf))), u);
}
__device__ __forceinline__ uint4 rv_swiglu8(uint4 g, uint4 u) {
  uint4 r;
  const __half* gh = reinterpret_cast<const __half*>(&g);
  const __half* uh = reinterpret_cast<const __half*>(&u);
  __half* rh = reinterpret_cast<__half*>(&r);
#pragma unroll
  for (int i = 0; i < 8; ++i) rh[i] = rv_swiglu(gh[i], uh[i]);
  return r;
}
// D (16 x 8, s32) += A (16 x 32, u8) . B (32 x 8, s8)
__device__ __forceinline__ void rv_imma(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// D (16 x 8, s32) = A (16 x 32, u8) . B (32 x 8, s8): the first product of a chain, no accumulator to initialise
__device__ __forceinline__ void rv_imma_z(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}
// D (16 x 8, f32) += A (16 x 16, f16) . B (16 x 8, f16)
__device__ __forceinline__ void rv_hmma(float (&d)[4], const uint4 a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}


// Requests tile `tile` of the layer (the groups [gb, gb + gn) of it, with the cherry blocks if `cherry`)
// into ring slot `slot`; one thread calls it.
__device__ __forceinline__ void issue_tile(const RowvecParams& p, const uint8_t* tiles, unsigned char* stiles, uint32_t bar_full,
                                           int tile, int slot, int gb, int gn, bool cherry) {
  const uint8_t* src = tiles + (size_t)tile * p.tile_bytes;
  const uint32_t dst = rv_smem_u32(stiles) + (uint32_t)slot * p.slot_bytes;
  const uint32_t bar = bar_full + 8 * slot;
  if (p.ks == 1) {                       // the whole record, which is also the slot's layout
    rv_mbar_expect_tx(bar, (uint32_t)p.tile_bytes);
    for (uint32_t off = 0; off < (uint32_t)p.tile_bytes; off += 32768) {
      const uint32_t sz = (uint32_t)p.tile_bytes - off < 32768 ? (uint32_t)p.tile_bytes - off : 32768;
      rv_bulk_g2s(dst + off, src + off, sz, bar);
    }
    return;
  }
  const uint32_t gbytes = (uint32_t)gn * p.grp_bytes, sbytes = (uint32_t)gn * p.set_bytes;
  const uint32_t cbytes = cherry ? (uint32_t)p.ncb * 512u : 0u;
  rv_mbar_expect_tx(bar, gbytes + sbytes + cbytes);
  const uint8_t* gsrc = src + (size_t)gb * p.grp_bytes;
  for (uint32_t off = 0; off < gbytes; off += 32768) {
    const uint32_t sz = gbytes - off < 32768 ? gbytes - off : 32768;
    rv_bulk_g2s(dst + off, gsrc + off, sz, bar);
  }
  rv_bulk_g2s(dst + p.scal_off_s, src + p.scal_off + (size_t)gb * p.set_bytes, sbytes, bar);
  if (cbytes) rv_bulk_g2s(dst + p.cher_off_s, src + p.cher_off, cbytes, bar);
}

// BITS 3 | 4; SETS scale sets per 128 columns (2 for 64-wide groups); W working warps per CTA plus
// one warp that only issues the bulk copies (a bulk copy instruction blocks its thread while
// the copy queue is full, i.e. for most of the streaming time: that thread must not have other
// work); GPW groups of 128 columns a warp can own (its activations stay in 8 * GPW registers).
// MR = 1: one activation row (the row loop below collapses); MR = 4: p.M rows, 1..4.
template <int BITS, int SETS, int W, int GPW, int MR>
__global__ void __launch_bounds__((W + 1) * 32, 1) cq_rowvec_kernel(const RowvecParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_abort, s_last;
  constexpr int NTHR = (W + 1) * 32;
  constexpr int GRP_BYTES = 256 * BITS;      // 16 rows x 128 codes
  constexpr int PVW = (GPW + 1) / 2;         // octets of activations a lane stages (16 per group, 32 lanes)
  constexpr int XCH = GPW / 2 + 1;           // 16-byte pieces of the raw slice a lane loads
  constexpr float OFF = BITS == 4 ? 7.5f : 3.5f;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g8 = lane >> 2, t4 = lane & 3;

  __half* slice = reinterpret_cast<__half*>(smem + p.off_slice) + (size_t)warp * p.slice_halves;
  uint32_t* plane = reinterpret_cast<uint32_t*>(slice);      // the planes replace the raw slice once it has been read
  float* part = reinterpret_cast<float*>(smem + p.off_part);
  const uint32_t bar_full = rv_smem_u32(smem + p.off_bar);
  const uint32_t bar_empty = bar_full + 8 * RV_MAX_SLOTS;
  unsigned char* stiles = smem + p.off_tiles;

  // the layer this CTA works on, and its tiles of it
  int si = 0;
#pragma unroll
  for (int s = 1; s < RV_MAX_SEG; ++s)
    if (s < p.nseg && (int)blockIdx.x >= p.seg[s].cta0) si = s;
  const RowvecSeg& sg = p.seg[si];
  const int bseg = (int)blockIdx.x - sg.cta0;
  const int ks = p.ks;
  const int unit = ks == 1 ? bseg : bseg / ks;            // CTAs of a unit share tiles, each takes a part of the columns
  const int kpart = ks == 1 ? 0 : bseg - unit * ks;
  const int tile0 = unit * sg.tiles_q + min(unit, sg.tiles_r);
  const int nt = sg.tiles_q + (unit < sg.tiles_r ? 1 : 0);
  const int gb = kpart * p.NGp;                           // first group of this CTA's part
  const int NGl = min(p.NG - gb, p.NGp);                  // its groups
  const int S = p.slots;

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < S; ++s) {
      rv_mbar_init(bar_full + 8 * s, 1);
      rv_mbar_init(bar_empty + 8 * s, W);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == W) {
    // ---- copy warp.  Tiles are requested in order with at most `inflight` of them outstanding:
    // enough bytes in flight to keep HBM busy, but short queues in the memory system, because the
    // working warps' activation loads (issued after the dependency wait, in the middle of the
    // stream) wait behind whatever is outstanding.  A ring slot is re-used once every working warp
    // has released it.
    if (lane == 0) {
      asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
      const uint8_t* seg_tiles = sg.tiles;
      int slot = 0, lslot = 0;                      // slot of the tile to issue / of the tile `inflight` back
      uint32_t ephase = 0, lphase = 0;              // phases of the empty / full barriers waited on
      for (int next = 0; next < nt; ++next) {
        if (next >= p.inflight) {                   // tile next - inflight must have landed
          rv_mbar_wait(bar_full + 8 * lslot, lphase, &s_abort, p.status);
          if (++lslot == S) { lslot = 0; lphase ^= 1u; }
        }
        if (next >= S) {                            // the slot's previous tile must have been consumed
          rv_mbar_wait(bar_empty + 8 * slot, ephase, &s_abort, p.status);
        }
        issue_tile(p, seg_tiles, stiles, bar_full, tile0 + next, slot, gb, NGl, kpart == 0);
        if (++slot == S) { slot = 0; if (next >= S) ephase ^= 1u; }
      }
    }
  } else {
  // ---- this warp's groups (contiguous) and cherry block
  const uint16_t* seg_perm = sg.perm;
  const int gq = NGl / W, gr = NGl % W;
  const int ngw = gq + (warp < gr ? 1 : 0);
  const int gstart = warp * gq + min(warp, gr);              // within the CTA's part (= within its ring slots)
  const int g0 = gb + gstart;                                // within the layer
  const bool has_cherry = warp < p.ncb && kpart == 0;        // cherry block `warp`
  // the original columns the warp's compact columns span: [lo, hi]; the slice starts at lo rounded down to 8
  int lo8 = 0, nchunk = 0;
  if (ngw > 0) {
    const int kc0 = g0 * 128, kc1 = min(p.K - p.C, (g0 + ngw) * 128) - 1;
    const int lo = seg_perm[kc0], hi = seg_perm[kc1];
    lo8 = lo & ~7;
    nchunk = (hi - lo8) / 8 + 1;
  }
  // column lists of the octets this lane stages (octet lane + 32 u of the warp's groups), turned into
  // byte offsets inside the slice here, ahead of the wait: two 16-bit fields per word, no field
  // underflows (every column is >= lo8) or overflows (the slice is a few hundred halves).  Padding
  // columns (= K) land on the zero slot at slice[K - lo8], which only the last group's warp has.
  uint4 pv[PVW];
#pragma unroll
  for (int u = 0; u < PVW; ++u) {
    const int ol = lane + 32 * u;
    uint4 c = make_uint4(0, 0, 0, 0);
    if (ol < ngw * 16) {
      c = *reinterpret_cast<const uint4*>(seg_perm + ((size_t)g0 * 16 + ol) * 8);
      const uint32_t sub = (uint32_t)lo8 * 0x10001u;
      c.x = (c.x - sub) * 2u; c.y = (c.y - sub) * 2u; c.z = (c.z - sub) * 2u; c.w = (c.w - sub) * 2u;
    }
    pv[u] = c;
  }
  const bool owns_tail = ngw > 0 && g0 + ngw == p.NG;       // the warp whose last group may hold padding columns
  int ccol = -1;
  if (has_cherry && lane < 16 && warp * 16 + lane < p.C) ccol = sg.cidx[warp * 16 + lane];
  const bool gated = p.x2 != nullptr;
  const bool x_aligned = ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.x2) | (uintptr_t)(p.ldx * 2)) & 15) == 0;
  // 16 bytes / one element of the activations at element offset `at` of the matrix
  auto ld8 = [&](size_t at) {
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(p.x + at));
    return gated ? rv_swiglu8(v, __ldcg(reinterpret_cast<const uint4*>(p.x2 + at))) : v;
  };
  auto ld1 = [&](size_t at) {
    const __half v = __ldcg(p.x + at);
    return gated ? rv_swiglu(v, __ldcg(p.x2 + at)) : v;
  };

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // What a lane keeps of the activations.  The integer MMA's B operand has 8 columns: column 2 m holds
  // the high plane of activation row m, column 2 m + 1 its low plane, so up to four rows ride in the MMAs
  // one row needs.  A lane's B column is g8 (it holds the planes of row g8 >> 1), and the sums it gets back
  // are those of row t4: sx16 / cq are row t4's terms.
  float sx16[GPW], cq[GPW][SETS];
  uint32_t xb[GPW][8];
  uint32_t cb0 = 0, cb1 = 0;
#pragma unroll
  for (int gi = 0; gi < GPW; ++gi) {
    sx16[gi] = 0.f;
#pragma unroll
    for (int s = 0; s < SETS; ++s) cq[gi][s] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) xb[gi][e] = 0u;
  }

  const int Mrows = MR == 1 ? 1 : p.M;
  // ---- the warp's slice of row m -> its shared-memory slice (coalesced 16-byte loads), cherry activations.
  // The loads of row m + 1 are in flight while row m is gathered and quantised.
  uint4 xv[XCH];
  uint32_t xcv_next = 0;
  if (x_aligned) {
#pragma unroll
    for (int c = 0; c < XCH; ++c) {
      const int ch = lane + 32 * c;
      xv[c] = make_uint4(0, 0, 0, 0);
      if (ch < nchunk) xv[c] = ld8((size_t)lo8 + 8 * ch);
    }
  }
  if (ccol >= 0) xcv_next = (uint32_t)__half_as_ushort(ld1((size_t)ccol));
#pragma unroll 1
  for (int m = 0; m < Mrows; ++m) {
  const uint32_t xcv = xcv_next;
  if (x_aligned) {
#pragma unroll
    for (int c = 0; c < XCH; ++c) {
      const int ch = lane + 32 * c;
      if (ch < nchunk) reinterpret_cast<uint4*>(slice)[ch] = xv[c];
    }
  } else {
    const size_t xr = (size_t)m * p.ldx + lo8;
    for (int i = lane; i < nchunk * 8; i += 32) slice[i] = ld1(xr + i);
  }
  if (MR > 1 && m + 1 < Mrows) {
    const size_t xn = (size_t)(m + 1) * p.ldx;
    if (x_aligned) {
#pragma unroll
      for (int c = 0; c < XCH; ++c) {
        const int ch = lane + 32 * c;
        if (ch < nchunk) xv[c] = ld8(xn + lo8 + 8 * ch);
      }
    }
    if (ccol >= 0) xcv_next = (uint32_t)__half_as_ushort(ld1(xn + ccol));
  }
  if (owns_tail && lane == 0) slice[p.K - lo8] = __float2half(0.f);   // zero slot for padding columns
  __syncwarp();

  // ---- gather every octet of this lane first: the planes written below re-use the slice's memory
  uint32_t xg[PVW][4];
#pragma unroll
  for (int u = 0; u < PVW; ++u) {
    const uint32_t pw[4] = {pv[u].x, pv[u].y, pv[u].z, pv[u].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t a = *reinterpret_cast<const unsigned short*>(reinterpret_cast<const unsigned char*>(slice) + (pw[i] & 0xFFFFu));
      const uint32_t b = *reinterpret_cast<const unsigned short*>(reinterpret_cast<const unsigned char*>(slice) + (pw[i] >> 16));
      xg[u][i] = __byte_perm(a, b, 0x5410);
    }
  }
  __syncwarp();
  // ---- quantise: one step size per group (16 consecutive lanes), two signed-byte planes, stored
  // where the B-fragment lanes pick them up with two 16-byte loads per group
#pragma unroll
  for (int u = 0; u < PVW; ++u) {
    const int ol = lane + 32 * u;
    float v[8];
    float mx = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&xg[u][i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
      mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
#pragma unroll
    for (int s = 1; s < 16; s <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, s));
    const float step = mx * (1.0f / 16256.0f);
    const float inv = mx > 0.f ? __fdividef(16256.0f, mx) : 0.f;
    // q = rint(v * inv) as 128 hi + lo with hi = rint(q / 128) in [-127, 127], lo in [-64, 64], all in
    // fp32 on the (full-rate) FMA pipe: adding 1.5 * 2^23 rounds to an integer and leaves it in the low
    // mantissa bits, so the low byte of the float's bit pattern is the signed byte wanted; no
    // float-to-int conversions, no integer arithmetic.  Any exact split q = 128 hi + lo gives the
    // same integer sums downstream.
    constexpr float MAGIC = 12582912.0f;
    uint32_t hi[8], lo[8];
    float sq = 0.f;                                  // sums of q stay exact in fp32 (< 2^24)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float qf = fmaf(v[i], inv, MAGIC) - MAGIC;          // |q| <= 16256 + 1 (approximate reciprocal)
      const float hm = fmaf(qf, 1.0f / 128.0f, MAGIC);
      const float lm = fmaf(hm - MAGIC, -128.0f, qf) + MAGIC;
      hi[i] = __float_as_uint(hm);
      lo[i] = __float_as_uint(lm);
      sq += qf;
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
    const float sq_other = __shfl_xor_sync(0xFFFFFFFFu, sq, 8);
    const float sq_a = (lane & 8) ? sq_other : sq, sq_b = (lane & 8) ? sq : sq_other;   // first / second half
    if (ol < ngw * 16) {
      // word wI (columns 4 wI .. 4 wI + 3 of the group) goes to [plane][t = wI & 3][chunk wI >> 3][(wI >> 2) & 1]
      const int gi = ol >> 4, oo = ol & 15;
      uint32_t* gp = plane + gi * 64;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int wI = 2 * oo + k;
        const int pos = (wI & 3) * 8 + (wI >> 3) * 2 + ((wI >> 2) & 1);
        gp[pos] = hw[k];
        gp[32 + pos] = lw[k];
      }
    }
    // the lanes that will receive row m's sums keep its terms of both groups of this round
    // (lanes 0-15 quantised group 2u, lanes 16-31 group 2u + 1)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (2 * u + h < GPW) {
        const float st = __shfl_sync(0xFFFFFFFFu, step, 16 * h);
        const float qa = __shfl_sync(0xFFFFFFFFu, sq_a, 16 * h), qb = __shfl_sync(0xFFFFFFFFu, sq_b, 16 * h);
        if (t4 == m) {
          sx16[2 * u + h] = st * (1.0f / 16.0f);
          if (SETS == 2) {
            cq[2 * u + h][0] = -OFF * st * qa;
            cq[2 * u + h][SETS - 1] = -OFF * st * qb;
          } else {
            cq[2 * u + h][0] = -OFF * st * (qa + qb);
          }
        }
      }
    }
  }
  __syncwarp();
  // B fragments of row m: lanes with g8 == 2 m take the high plane, g8 == 2 m + 1 the low plane
  const bool mine = (g8 >> 1) == m;
#pragma unroll
  for (int gi = 0; gi < GPW; ++gi) {
    if (mine && gi < ngw) {
      const uint4* src = reinterpret_cast<const uint4*>(plane + gi * 64 + (g8 & 1) * 32 + t4 * 8);
      const uint4 a = src[0], b = src[1];
      xb[gi][0] = a.x; xb[gi][1] = a.y; xb[gi][2] = a.z; xb[gi][3] = a.w;
      xb[gi][4] = b.x; xb[gi][5] = b.y; xb[gi][6] = b.z; xb[gi][7] = b.w;
    }
  }
  // cherry B fragment (16 x 8 halves, column 2 m = row m's cherry activations, odd columns zero):
  // b0 = x_c[2t], x_c[2t + 1]; b1 = x_c[8 + 2t], x_c[9 + 2t]
  if (has_cherry) {
    const uint32_t v0 = __shfl_sync(0xFFFFFFFFu, xcv, 2 * t4), v1 = __shfl_sync(0xFFFFFFFFu, xcv, 2 * t4 + 1);
    const uint32_t v2 = __shfl_sync(0xFFFFFFFFu, xcv, 8 + 2 * t4), v3 = __shfl_sync(0xFFFFFFFFu, xcv, 9 + 2 * t4);
    if (g8 == 2 * m) {
      cb0 = v0 | (v1 << 16);
      cb1 = v2 | (v3 << 16);
    }
  }
  __syncwarp();                                       // the next row re-uses the slice
  }   // activation rows

  // ---- tiles.  Addresses: one base per kind (codes, scales, cherry, partial sums) computed here,
  // the ring slot's offset kept incrementally, everything else is a compile-time displacement.
  const unsigned char* gp0 = stiles + (size_t)gstart * GRP_BYTES + lane * 16;
  const unsigned char* gq0 = stiles + (size_t)gstart * GRP_BYTES + 512 + lane * (BITS == 4 ? 16 : 8);
  const unsigned char* sp0 = stiles + p.scal_off_s + (gstart * SETS * 8 + g8) * 4;
  const unsigned char* cp0 = stiles + p.cher_off_s + warp * 512 + lane * 16;
  float* pp = part + (warp * Mrows + t4) * 16 + g8;
  int slot = 0;
  uint32_t slot_off = 0, phase = 0;
#pragma unroll 1
  for (int i = 0; i < nt; ++i) {
    rv_mbar_wait(bar_full + 8 * slot, phase, &s_abort, p.status);
    float acc0 = 0.f, acc1 = 0.f;                            // rows g8 and g8 + 8 of the tile
#pragma unroll
    for (int gi = 0; gi < GPW; ++gi) {
      if (gi < ngw) {                                        // warp-uniform
        const unsigned char* gp = gp0 + slot_off + gi * GRP_BYTES;
        const unsigned char* gq = gq0 + slot_off + gi * GRP_BYTES;
        int dP[SETS][4], dH[SETS][4];
        if (BITS == 4) {
          const uint4 w0 = *reinterpret_cast<const uint4*>(gp);
          const uint4 w1 = *reinterpret_cast<const uint4*>(gq);
          const uint32_t wa[4] = {w0.x, w0.y, w0.z, w0.w}, wc[4] = {w1.x, w1.y, w1.z, w1.w};
          uint32_t aP[4], aH[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) { aP[j] = wa[j] & 0x0F0F0F0Fu; aH[j] = wa[j] & 0xF0F0F0F0u; }
          rv_imma_z(dP[0], aP, xb[gi][0], xb[gi][1]);        // columns 0..31
          rv_imma_z(dH[0], aH, xb[gi][2], xb[gi][3]);        // columns 32..63, as 16 u
#pragma unroll
          for (int j = 0; j < 4; ++j) { aP[j] = wc[j] & 0x0F0F0F0Fu; aH[j] = wc[j] & 0xF0F0F0F0u; }
          if (SETS == 1) {
            rv_imma(dP[0], aP, xb[gi][4], xb[gi][5]);        // columns 64..95
            rv_imma(dH[0], aH, xb[gi][6], xb[gi][7]);        // columns 96..127
          } else {
            rv_imma_z(dP[SETS - 1], aP, xb[gi][4], xb[gi][5]);
            rv_imma_z(dH[SETS - 1], aH, xb[gi][6], xb[gi][7]);
          }
        } else {
          const uint4 w0 = *reinterpret_cast<const uint4*>(gp);
          const uint2 w1 = *reinterpret_cast<const uint2*>(gq);
          const uint32_t ws[2][3] = {{w0.x, w0.y, w0.z}, {w0.w, w1.x, w1.y}};
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const uint32_t A = ws[s][0], B = ws[s][1], Cw = ws[s][2];
            const uint32_t A3 = A >> 3, B2 = B >> 2, C1 = Cw >> 1;
            uint32_t aP[4], aH[4];
            aP[0] = A & 0x07070707u;  aH[0] = A & 0x70707070u;
            aP[1] = B & 0x07070707u;  aH[1] = B & 0x70707070u;
            aP[2] = Cw & 0x07070707u; aH[2] = Cw & 0x70707070u;
            aP[3] = (A3 & 0x01010101u) | (B2 & 0x02020202u) | (C1 & 0x04040404u);
            aH[3] = (A3 & 0x10101010u) | (B2 & 0x20202020u) | (C1 & 0x40404040u);
            if (s == 0 || SETS == 2) {                       // the first product into an accumulator
              rv_imma_z(dP[s * (SETS - 1)], aP, xb[gi][4 * s], xb[gi][4 * s + 1]);   // columns 64 s .. 64 s + 31
              rv_imma_z(dH[s * (SETS - 1)], aH, xb[gi][4 * s + 2], xb[gi][4 * s + 3]);   // columns 64 s + 32 .. 64 s + 63, as 16 u
            } else {
              rv_imma(dP[0], aP, xb[gi][4 * s], xb[gi][4 * s + 1]);
              rv_imma(dH[0], aH, xb[gi][4 * s + 2], xb[gi][4 * s + 3]);
            }
          }
        }
        // lanes with t4 == 0 hold column 0 (hi sums) and column 1 (lo sums) of rows g8, g8 + 8
#pragma unroll
        for (int s = 0; s < SETS; ++s) {
          const __half2 sc2 = *reinterpret_cast<const __half2*>(sp0 + slot_off + (gi * SETS + s) * 32);
          const float2 scf = __half22float2(sc2);
          const int t0 = ((dP[s][0] * 128 + dP[s][1]) << 4) + (dH[s][0] * 128 + dH[s][1]);
          const int t1 = ((dP[s][2] * 128 + dP[s][3]) << 4) + (dH[s][2] * 128 + dH[s][3]);
          acc0 = fmaf(scf.x, fmaf((float)t0, sx16[gi], cq[gi][s]), acc0);
          acc1 = fmaf(scf.y, fmaf((float)t1, sx16[gi], cq[gi][s]), acc1);
        }
      }
    }
    if (has_cherry) {
      const uint4 a = *reinterpret_cast<const uint4*>(cp0 + slot_off);
      float dc[4] = {0.f, 0.f, 0.f, 0.f};
      rv_hmma(dc, a, cb0, cb1);
      acc0 += dc[0];
      acc1 += dc[2];
    }
    if (t4 < Mrows) {                                        // the sums of activation row t4
      pp[0] = acc0;
      pp[8] = acc1;
    }
    pp += W * Mrows * 16;
    if (i + S < nt) {
      // ring: this warp is done with the slot; the copy warp refills it once every warp is
      __syncwarp();
      if (lane == 0) rv_mbar_arrive(bar_empty + 8 * slot);
    }
    ++slot;
    slot_off += (uint32_t)p.slot_bytes;
    if (slot == S) { slot = 0; slot_off = 0; phase ^= 1u; }
  }
  }   // working warps
  __syncthreads();
  // ---- the warps' partial sums of every row, in warp order
  const int row0 = tile0 * 16;
  __half* y = sg.y;
  const int N = sg.N;
  const int M = MR == 1 ? 1 : p.M;
  if (ks == 1) {
    for (int idx = tid; idx < nt * 16 * M; idx += NTHR) {
      const int tl = idx / (16 * M), rem = idx - tl * 16 * M;
      const int m = rem >> 4, r = rem & 15;
      const int row = row0 + tl * 16 + r;
      if (row < N) {
        const float* pp = part + ((size_t)tl * W * M + m) * 16 + r;
        __half* yo = y + (size_t)m * p.ldy + row;
        float acc = p.accumulate ? __half2float(*yo) : 0.f;
#pragma unroll
        for (int w = 0; w < W; ++w) acc += pp[w * M * 16];
        *yo = __float2half_rn(acc);
      }
    }
  } else {
    // this part's sums -> global; the CTA of the unit that arrives last adds the parts in part order
    const size_t per_part = (size_t)sg.NT * 16 * M;
    float* mine = sg.work + kpart * per_part + (size_t)tile0 * 16 * M;
    for (int idx = tid; idx < nt * 16 * M; idx += NTHR) {
      const int tl = idx / (16 * M), rem = idx - tl * 16 * M;
      const float* pp = part + ((size_t)tl * W * M + (rem >> 4)) * 16 + (rem & 15);
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < W; ++w) acc += pp[w * M * 16];
      mine[idx] = acc;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&sg.counters[tile0], 1u) == (unsigned int)(ks - 1);
    __syncthreads();
    if (s_last) {
      __threadfence();
      const float* all = sg.work + (size_t)tile0 * 16 * M;
      for (int idx = tid; idx < nt * 16 * M; idx += NTHR) {
        const int tl = idx / (16 * M), rem = idx - tl * 16 * M;
        const int m = rem >> 4, r = rem & 15;
        const int row = row0 + tl * 16 + r;
        if (row < N) {
          __half* yo = y + (size_t)m * p.ldy + row;
          float acc = p.accumulate ? __half2float(*yo) : 0.f;
          for (int j = 0; j < ks; ++j) acc += __ldcg(all + j * per_part + idx);
          *yo = __float2half_rn(acc);
        }
      }
      if (tid == 0) sg.counters[tile0] = 0u;               // ready for the next launch
    }
  }
  if (p.gather) {
    // every CTA has stored its rows of the local slice; the last one to get here exchanges the slices
    uint8_t* own = nullptr;
#pragma unroll
    for (int r = 0; r < cq_peer::MAX_RANKS; ++r)
      if (r == p.peer.rank) own = p.peer.region[r];
    unsigned int* done = reinterpret_cast<unsigned int*>(own + cq_peer::DONE_OFF);
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(done, 1u) == gridDim.x - 1u;
    __syncthreads();
    if (s_last) {
      __threadfence();
      cq_peer::exchange<NTHR>(p.peer, &s_abort);          // (s_abort has no other use any more: every copy has landed)
      if (tid == 0) *done = 0u;                            // ready for the next launch
    }
  }
}

// ------------------------------------------------------------------ layout kernels
struct RlayerDev {
  uint8_t* tiles; uint16_t* perm; uint16_t* cidx;
  int bits, K, N, C, G, Kc, NG, sets, Cp, NT, tile_bytes, scal_off, cher_off;
};

RlayerDev rl_view(const cq_rlayer* L) {
  RlayerDev d;
  uint8_t* b = (uint8_t*)L->blob;
  d.tiles = b + L->off_tiles;
  d.perm = (uint16_t*)(b + L->off_perm);
  d.cidx = (uint16_t*)(b + L->off_cidx);
  d.bits = L->bits; d.K = L->K; d.N = L->N; d.C = L->C; d.G = L->G; d.Kc = L->Kc; d.NG = L->NG;
  d.sets = L->sets; d.Cp = L->Cp; d.NT = L->NT; d.tile_bytes = L->tile_bytes;
  d.scal_off = L->NG * 256 * L->bits;
  d.cher_off = d.scal_off + L->NG * L->sets * 32;
  return d;
}

// Layout of one group block (16 rows x 128 compact columns) as the kernel's lanes read it.
// Lane (g8, t) = 4 g8 + t; A-fragment register j of a 32-column chunk holds, as bytes b = 0..3,
// row g8 + 8 (j & 1), columns 16 (j >> 1) + 4 t + b of the chunk.
//   4-bit: two 16-byte loads per lane, [load l][lane][16 B]; word j of load l = register j of
//     chunk 2 l in the low nibbles and of chunk 2 l + 1 in the high nibbles.
//   3-bit: per 64-column half s the words A, B, C = wi 0, 1, 2, stored as [lane][16 B] =
//     {A0, B0, C0, A1} and, from byte 512, [lane][8 B] = {B1, C1}.  Word wi holds register wi of
//     chunk 2 s in bits 0-2 and of chunk 2 s + 1 in bits 4-6 of its bytes; register 3 is spread
//     as bit planes: code bit wi of chunk 2 s (chunk 2 s + 1) in bit 3 (bit 7) of word wi.
__device__ __forceinline__ int rl3_word_off(int lane, int widx) {     // widx = 3 s + wi, 0..5
  return widx < 4 ? lane * 16 + widx * 4 : 512 + lane * 8 + (widx - 4) * 4;
}
// Byte offset (inside the group block) of the word that holds bit i of code (row rl, column kk), and the bit.
__device__ __forceinline__ void rl_bit_pos(int bits, int rl, int kk, int i, int* off, int* bit) {
  const int chunk = kk >> 5, k32 = kk & 31;
  const int j = ((k32 >> 4) << 1) | (rl >> 3);
  const int t = (k32 & 15) >> 2, b = k32 & 3;
  const int lane = (rl & 7) * 4 + t;
  if (bits == 4) {
    *off = (chunk >> 1) * 512 + lane * 16 + j * 4;
    *bit = 8 * b + 4 * (chunk & 1) + i;
  } else {
    const int s = chunk >> 1;
    if (j < 3) {
      *off = rl3_word_off(lane, 3 * s + j);
      *bit = 8 * b + 4 * (chunk & 1) + i;
    } else {
      *off = rl3_word_off(lane, 3 * s + i);
      *bit = 8 * b + ((chunk & 1) ? 7 : 3);
    }
  }
}

// one thread per 32-bit word of a group block: gathers the codes the word holds
__global__ void rl_prepare_codes_kernel(RlayerDev d, const uint8_t* __restrict__ q) {
  const int wpg = 64 * d.bits;                               // words per group block
  const size_t total = (size_t)d.NT * d.NG * wpg;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int wq = (int)(idx % wpg);
    const size_t rest = idx / wpg;
    const int gg = (int)(rest % d.NG), tile = (int)(rest / d.NG);
    int lane, widx;                                          // which lane's word
    if (d.bits == 4) { lane = (wq >> 2) & 31; widx = (wq >> 7) * 4 + (wq & 3); }          // widx = 4 l + j
    else if (wq < 128) { lane = wq >> 2; widx = wq & 3; }
    else { lane = (wq - 128) >> 1; widx = 4 + ((wq - 128) & 1); }
    const int byte_off = d.bits == 4 ? (wq >> 7) * 512 + lane * 16 + (wq & 3) * 4 : rl3_word_off(lane, widx);
    const int g8 = lane >> 2, t = lane & 3;
    uint32_t word = 0;
    auto code = [&](int rl, int kk) -> uint32_t {
      const int n = tile * 16 + rl, kc = gg * 128 + kk;
      return (n < d.N && kc < d.Kc) ? cq_ref_code(q, d.bits, kc, n, d.N) : 0u;
    };
    if (d.bits == 4) {
      const int l = widx >> 2, j = widx & 3;
      const int rl = g8 + 8 * (j & 1), kb = 16 * (j >> 1) + 4 * t;
      for (int b = 0; b < 4; ++b) {
        word |= code(rl, 32 * (2 * l) + kb + b) << (8 * b);
        word |= code(rl, 32 * (2 * l + 1) + kb + b) << (8 * b + 4);
      }
    } else {
      const int s = widx / 3, wi = widx % 3;
      const int rl = g8 + 8 * (wi & 1), kb = 16 * (wi >> 1) + 4 * t;          // register wi
      const int rl3 = g8 + 8, kb3 = 16 + 4 * t;                               // register 3
      for (int b = 0; b < 4; ++b) {
        word |= code(rl, 32 * (2 * s) + kb + b) << (8 * b);
        word |= code(rl, 32 * (2 * s + 1) + kb + b) << (8 * b + 4);
        word |= ((code(rl3, 32 * (2 * s) + kb3 + b) >> wi) & 1u) << (8 * b + 3);
        word |= ((code(rl3, 32 * (2 * s + 1) + kb3 + b) >> wi) & 1u) << (8 * b + 7);
      }
    }
    *reinterpret_cast<uint32_t*>(d.tiles + (size_t)tile * d.tile_bytes + (size_t)gg * wpg * 4 + byte_off) = word;
  }
}

// scales, cherry values, column permutation and cherry list
__global__ void rl_prepare_rest_kernel(RlayerDev d, const __half* __restrict__ scales, const __half* __restrict__ cw,
                                       const int16_t* __restrict__ ci) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int ngr = (d.Kc + d.G - 1) / d.G;            // scale rows of the reference
  const size_t rows = (size_t)d.NT * 16;
  // scales: [group][set][g8][row g8, row g8 + 8]
  for (size_t idx = t0; idx < rows * d.NG * d.sets; idx += stride) {
    const int n = (int)(idx % rows);
    const int gs = (int)(idx / rows);
    const int kc = (gs / d.sets) * 128 + (gs % d.sets) * 64;
    const int gi = kc / d.G;
    const bool real = n < d.N && kc < d.Kc && gi < ngr;
    __half* sp = reinterpret_cast<__half*>(d.tiles + (size_t)(n >> 4) * d.tile_bytes + d.scal_off) +
                 ((size_t)gs * 8 + (n & 7)) * 2 + ((n >> 3) & 1);
    *sp = real ? scales[(size_t)gi * d.N + n] : __float2half(0.f);
  }
  // cherry A fragments (m16n8k16): register j of lane (g8, t): row g8 + 8 (j & 1), columns 8 (j >> 1) + 2 t + {0, 1}
  for (size_t idx = t0; idx < rows * d.Cp; idx += stride) {
    const int n = (int)(idx % rows), c = (int)(idx / rows);
    const int rl = n & 15, cc = c & 15;
    const int lane = (rl & 7) * 4 + ((cc & 7) >> 1), j = ((cc >> 3) << 1) | (rl >> 3);
    __half* cp = reinterpret_cast<__half*>(d.tiles + (size_t)(n >> 4) * d.tile_bytes + d.cher_off + (size_t)(c >> 4) * 512 +
                                           lane * 16 + j * 4) + (cc & 1);
    *cp = (n < d.N && c < d.C) ? cw[(size_t)c * d.N + n] : __float2half(0.f);
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
  for (size_t idx = t0; idx < (size_t)d.Cp; idx += stride) d.cidx[idx] = idx < (size_t)d.C ? (uint16_t)ci[idx] : (uint16_t)d.K;
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
    for (int e = 0; e < 8; ++e) {
      const int kc = 8 * o + e;
      const uint8_t* gp = d.tiles + (size_t)(n >> 4) * d.tile_bytes + (size_t)(kc >> 7) * 256 * d.bits;
      uint32_t v = 0;
      for (int i = 0; i < d.bits; ++i) {
        int off, bit;
        rl_bit_pos(d.bits, n & 15, kc & 127, i, &off, &bit);
        v |= ((*reinterpret_cast<const uint32_t*>(gp + off) >> bit) & 1u) << i;
      }
      u[e] = v;
    }
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
    const int gs = (kc >> 7) * d.sets + ((kc >> 6) & (d.sets - 1));
    const __half* sp = reinterpret_cast<const __half*>(d.tiles + (size_t)(n >> 4) * d.tile_bytes + d.scal_off) +
                       ((size_t)gs * 8 + (n & 7)) * 2 + ((n >> 3) & 1);
    scales[(size_t)gi * d.N + n] = *sp;
  }
  for (size_t idx = t0; idx < (size_t)d.N * d.C; idx += stride) {
    const int n = (int)(idx % d.N), c = (int)(idx / d.N);
    const int rl = n & 15, cc = c & 15;
    const int lane = (rl & 7) * 4 + ((cc & 7) >> 1), j = ((cc >> 3) << 1) | (rl >> 3);
    const __half* cp = reinterpret_cast<const __half*>(d.tiles + (size_t)(n >> 4) * d.tile_bytes + d.cher_off +
                                                       (size_t)(c >> 4) * 512 + lane * 16 + j * 4) + (cc & 1);
    cw[(size_t)c * d.N + n] = *cp;
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

// Kernel shapes of the product: 16 working warps (+ the copy warp: 96 registers per thread) that own up to 2
// or up to 4 groups each, i.e. up to 64 groups per CTA; wider layers are split along K among several CTAs
// per tile (cq_rlayer.ksplit), which keeps every CTA inside these shapes.  0 = no shape holds the layer.
constexpr int RV_W = 16;
inline int rv_part_groups(const cq_rlayer* L) { return (L->NG + L->ksplit - 1) / L->ksplit; }   // groups a CTA works on
inline int rv_gpw_for(const cq_rlayer* L) {
  if (L->ksplit < 1 || L->ksplit > RV_MAX_KSPLIT) return 0;
  const int need = (rv_part_groups(L) + RV_W - 1) / RV_W;
  return need <= 2 ? 2 : (need <= 4 ? 4 : 0);
}

template <int W, int GPW>
RowvecFn rv_pick(int bits, int sets, int M = 1) {
  if (M == 1) {
    if (bits == 4) return cq_rowvec_kernel<4, 1, W, GPW, 1>;
    return sets == 1 ? cq_rowvec_kernel<3, 1, W, GPW, 1> : cq_rowvec_kernel<3, 2, W, GPW, 1>;
  }
  if (bits == 4) return cq_rowvec_kernel<4, 1, W, GPW, RV_MAX_ROWS>;
  return sets == 1 ? cq_rowvec_kernel<3, 1, W, GPW, RV_MAX_ROWS> : cq_rowvec_kernel<3, 2, W, GPW, RV_MAX_ROWS>;
}

// Plan of one launch over `n` layers that share the activation row (same bits, K, cherry count and
// group size, hence the same tile record size): how the CTAs are divided among the layers, the
// shared-memory sections, the ring.  W working warps own up to GPW groups each.  Fills the launch
// parameters that do not depend on the call.  Returns a status code.
int rv_plan(int W, int GPW, const cq_rlayer* const* Ls, int n, int M, const RvDevice& di,
            RowvecParams* p, int* grid_out, int* smem_out) {
  if (n < 1 || n > RV_MAX_SEG || M < 1 || M > RV_MAX_ROWS) return CQ_ERR_BAD_ARG;
  const cq_rlayer* L = Ls[0];
  for (int i = 1; i < n; ++i)
    if (Ls[i]->bits != L->bits || Ls[i]->K != L->K || Ls[i]->C != L->C || Ls[i]->G != L->G || Ls[i]->ksplit != L->ksplit) return CQ_ERR_BAD_SHAPE;
  const int ks = L->ksplit, ngp = rv_part_groups(L);
  if (ks < 1 || ks > RV_MAX_KSPLIT) return CQ_ERR_UNSUPPORTED;
  if ((ngp + W - 1) / W > GPW) return CQ_ERR_UNSUPPORTED;
  if (L->Cp / 16 > W) return CQ_ERR_UNSUPPORTED;
  if (GPW * 128 + L->C + 8 > (GPW / 2 + 1) * 256) return CQ_ERR_UNSUPPORTED;   // a warp's slice of x: XCH pieces per lane
  // units (ks CTAs sharing their tiles) per layer: every layer at least one, the rest to whichever layer has
  // the most tiles per unit
  const int units_avail = di.sms / ks;
  long long total = 0;
  for (int i = 0; i < n; ++i) total += Ls[i]->NT;
  int ctas[RV_MAX_SEG];                           // units per layer
  int grid = 0;
  if (total <= units_avail) {
    for (int i = 0; i < n; ++i) { ctas[i] = Ls[i]->NT; grid += ctas[i]; }
  } else {
    if (units_avail < n) return CQ_ERR_NO_DEVICE;
    for (int i = 0; i < n; ++i) {
      ctas[i] = (int)((long long)units_avail * Ls[i]->NT / total);
      if (ctas[i] < 1) ctas[i] = 1;
      grid += ctas[i];
    }
    while (grid > units_avail) {                 // (rounding up the small layers can overshoot)
      int big = 0;
      for (int i = 1; i < n; ++i) if (ctas[i] > ctas[big]) big = i;
      --ctas[big]; --grid;
    }
    for (; grid < units_avail; ++grid) {
      int worst = -1, worst_t = 0;
      for (int i = 0; i < n; ++i) {
        const int t = (Ls[i]->NT + ctas[i] - 1) / ctas[i];
        if (ctas[i] < Ls[i]->NT && t > worst_t) { worst = i; worst_t = t; }
      }
      if (worst < 0) break;
      ++ctas[worst];
    }
  }
  grid *= ks;
  int nt_max = 0, cta0 = 0;
  for (int i = 0; i < n; ++i) {
    RowvecSeg& sg = p->seg[i];
    sg.N = Ls[i]->N;
    sg.NT = Ls[i]->NT;
    sg.cta0 = cta0;
    sg.tiles_q = Ls[i]->NT / ctas[i];
    sg.tiles_r = Ls[i]->NT % ctas[i];
    const int t = (Ls[i]->NT + ctas[i] - 1) / ctas[i];
    if (t > nt_max) nt_max = t;
    cta0 += ctas[i] * ks;
  }
  p->nseg = n;
  p->K = L->K; p->C = L->C; p->NG = L->NG; p->ncb = L->Cp / 16;
  p->tile_bytes = L->tile_bytes;
  p->grp_bytes = 256 * L->bits;
  p->set_bytes = L->sets * 32;
  p->scal_off = L->NG * p->grp_bytes;
  p->cher_off = p->scal_off + L->NG * p->set_bytes;
  p->ks = ks; p->NGp = ngp;
  p->scal_off_s = ngp * p->grp_bytes;
  p->cher_off_s = p->scal_off_s + ngp * p->set_bytes;
  p->slot_bytes = p->cher_off_s + p->ncb * 512;        // ks == 1: the record itself (ngp == NG)
  // a warp's staging area: the raw slice (its column range + alignment slack + zero slot), later its planes
  const int gmax = (ngp + W - 1) / W;
  p->slice_halves = rv_align(gmax * 128 + L->C + 8 + 8 + 8, 8);
  if (p->slice_halves < gmax * 128) p->slice_halves = gmax * 128;     // planes: 256 bytes per group
  int off = 0;
  p->off_slice = off; off = rv_align(off + W * p->slice_halves * 2, 16);
  p->off_part = off;  off = rv_align(off + nt_max * W * M * 16 * 4, 16);
  p->off_bar = off;   off = rv_align(off + 2 * RV_MAX_SLOTS * 8, 128);
  p->off_tiles = off;
  int budget = di.max_smem - 1024;          // the kernel also has a small static allocation; keep clear of the limit
  int slots = (budget - off) / p->slot_bytes;
  if (slots > nt_max) slots = nt_max;
  if (slots > RV_MAX_SLOTS) slots = RV_MAX_SLOTS;
  if (slots < 1 || (slots < 2 && nt_max > 1)) return CQ_ERR_TOO_LARGE;
  p->slots = slots;
  // measured on B200: two tiles outstanding stream best when a CTA has several tiles (4096 -> 11008: 5.7 us
  // against 6.6 with one and 6.1 with three); with one or two tiles per CTA a single outstanding tile is faster
  const int inflight = nt_max >= 3 ? 2 : 1;
  p->inflight = inflight > slots ? slots : inflight;
  *grid_out = grid;
  *smem_out = off + slots * p->slot_bytes;
  return CQ_OK;
}

// One launch of a kernel whose warp count is W and whose warps can own GPW groups, over `n` layers
// that take the same activation row x; ys[i] receives layer i's output.
int rv_launch(RowvecFn fn, int W, int GPW, const cq_rlayer* const* Ls, int n, const __half* x, int ldx,
              __half* const* ys, int ldy, int M, int accumulate, uint32_t* status, cudaStream_t st,
              const cq_peer::PeerGatherParams* peer = nullptr, const __half* x2 = nullptr) {
  int dev = 0;
  CQ_CUDA_TRY(cudaGetDevice(&dev));
  const RvDevice di = rv_device(dev);
  if (!di.ok) return CQ_ERR_NO_DEVICE;
  RowvecParams p;
  int grid = 0, smem = 0;
  const int rc = rv_plan(W, GPW, Ls, n, M, di, &p, &grid, &smem);
  if (rc != CQ_OK) return rc;
  for (int i = 0; i < RV_MAX_SEG; ++i) {
    const int j = i < n ? i : 0;                 // unused entries repeat the first layer (never selected)
    const uint8_t* blob = (const uint8_t*)Ls[j]->blob;
    p.seg[i].tiles = blob + Ls[j]->off_tiles;
    p.seg[i].perm = (const uint16_t*)(blob + Ls[j]->off_perm);
    p.seg[i].cidx = (const uint16_t*)(blob + Ls[j]->off_cidx);
    p.seg[i].y = ys[j];
    p.seg[i].work = (float*)(blob + Ls[j]->off_work);
    p.seg[i].counters = (unsigned int*)(blob + Ls[j]->off_work + (size_t)Ls[j]->ksplit * Ls[j]->NT * 16 * RV_MAX_ROWS * sizeof(float));
    if (i >= n) { p.seg[i].N = 0; p.seg[i].cta0 = grid; p.seg[i].tiles_q = 0; p.seg[i].tiles_r = 0; }
  }
  p.x = x; p.x2 = x2; p.status = status;
  p.M = M; p.ldx = ldx; p.ldy = ldy;
  p.accumulate = accumulate;
  p.gather = peer ? 1 : 0;
  if (peer) p.peer = *peer; else p.peer = cq_peer::PeerGatherParams{};
  {
    // opt in to the dynamic shared memory this launch needs (remembered per kernel and device)
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, int> granted;
    std::lock_guard<std::mutex> lk(mu);
    int& have = granted[{(const void*)fn, dev}];
    if (smem > have) {
      CQ_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      have = smem;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3((W + 1) * 32);
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
  L->Cp = (C + 15) / 16 * 16;
  L->NT = (N + 15) / 16;
  L->tile_bytes = L->NG * 256 * bits + L->NG * L->sets * 32 + (L->Cp / 16) * 512;
  uint64_t off = 0;
  L->off_tiles = off;  off += (uint64_t)L->NT * L->tile_bytes;        off = (off + 255) / 256 * 256;
  L->off_perm = off;   off += (uint64_t)L->NG * 128 * 2;              off = (off + 255) / 256 * 256;
  L->off_cidx = off;   off += (uint64_t)(L->Cp > 0 ? L->Cp : 16) * 2; off = (off + 255) / 256 * 256;
  // layers of more than 64 groups are split along K among ksplit CTAs per tile; their partial sums
  // ([ksplit][NT][4 rows][16] fp32) and arrival counters ([NT] uint32) live behind the tables
  L->ksplit = (L->NG + 63) / 64;
  L->off_work = off;
  if (L->ksplit > 1) {
    off += (uint64_t)L->ksplit * L->NT * 16 * RV_MAX_ROWS * sizeof(float) + (uint64_t)L->NT * sizeof(uint32_t);
    off = (off + 255) / 256 * 256;
  }
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
  if (L->blob_bytes > L->off_work)
    CQ_CUDA_TRY(cudaMemsetAsync((uint8_t*)L->blob + L->off_work, 0, L->blob_bytes - L->off_work, st));
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

extern "C" int cq_rlayer_check(const cq_rlayer* L) {
  if (!L) return CQ_ERR_BAD_ARG;
  int dev = 0;
  CQ_CUDA_TRY(cudaGetDevice(&dev));
  const RvDevice di = rv_device(dev);
  if (!di.ok) return CQ_ERR_NO_DEVICE;
  const int gpw = rv_gpw_for(L);
  if (!gpw) return CQ_ERR_UNSUPPORTED;
  RowvecParams p;
  int grid = 0, smem = 0;
  return rv_plan(RV_W, gpw, &L, 1, RV_MAX_ROWS, di, &p, &grid, &smem);
}

extern "C" int cq_rlayers_matvec(const cq_rlayer* const* layers, int n_layers, const void* x, int ldx, void* const* ys, int ldy,
                                 int M, int accumulate, uint32_t* status_word, cq_stream_t stream) {
  if (!layers || !ys || !x || n_layers < 1 || n_layers > RV_MAX_SEG || M < 1) return CQ_ERR_BAD_ARG;
  if ((uintptr_t)x & 1) return CQ_ERR_BAD_ARG;
  int nmax = 0;
  for (int i = 0; i < n_layers; ++i) {
    if (!layers[i] || !layers[i]->blob || !ys[i] || ((uintptr_t)ys[i] & 1)) return CQ_ERR_BAD_ARG;
    if (layers[i]->N > nmax) nmax = layers[i]->N;
  }
  const cq_rlayer* L = layers[0];
  if (ldx < L->K || ldy < nmax) return CQ_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  // up to RV_MAX_ROWS activation rows per launch; more rows are walked in slices, each reading the weights again
  for (int m0 = 0; m0 < M; m0 += RV_MAX_ROWS) {
    const int rows = M - m0 < RV_MAX_ROWS ? M - m0 : RV_MAX_ROWS;
    const __half* xp = (const __half*)x + (size_t)m0 * ldx;
    __half* yp[RV_MAX_SEG];
    for (int i = 0; i < n_layers; ++i) yp[i] = (__half*)ys[i] + (size_t)m0 * ldy;
    int rc = CQ_ERR_UNSUPPORTED;
    switch (rv_gpw_for(L)) {
      case 2: rc = rv_launch(rv_pick<RV_W, 2>(L->bits, L->sets, rows), RV_W, 2, layers, n_layers, xp, ldx, yp, ldy, rows, accumulate, status_word, st); break;
      case 4: rc = rv_launch(rv_pick<RV_W, 4>(L->bits, L->sets, rows), RV_W, 4, layers, n_layers, xp, ldx, yp, ldy, rows, accumulate, status_word, st); break;
      default: break;
    }
    if (rc != CQ_OK) return rc;
  }
  return CQ_OK;
}

extern "C" int cq_rlayer_matvec_gather(const cq_rlayer* L, const void* x, int ldx, void* y_local, int M, void* const* regions,
                                       int world, int rank, size_t capacity, void* y_all, int timeout_ms,
                                       uint32_t* status_word, cq_stream_t stream) {
  if (!L || !L->blob || !x || !y_local || !y_all) return CQ_ERR_BAD_ARG;
  if (M < 1 || M > RV_MAX_ROWS || ldx < L->K) return CQ_ERR_BAD_ARG;
  if (((uintptr_t)x & 1) || ((uintptr_t)y_local & 7)) return CQ_ERR_BAD_ARG;
  cq_peer::PeerGatherParams pg;
  int rc = cq_peer::fill_params(&pg, regions, world, rank, capacity, y_local, y_all, M, L->N, timeout_ms, status_word);
  if (rc != CQ_OK) return rc;
  __half* yp = (__half*)y_local;
  cudaStream_t st = (cudaStream_t)stream;
  switch (rv_gpw_for(L)) {
    case 2: return rv_launch(rv_pick<RV_W, 2>(L->bits, L->sets, M), RV_W, 2, &L, 1, (const __half*)x, ldx, &yp, L->N, M, 0, status_word, st, &pg);
    case 4: return rv_launch(rv_pick<RV_W, 4>(L->bits, L->sets, M), RV_W, 4, &L, 1, (const __half*)x, ldx, &yp, L->N, M, 0, status_word, st, &pg);
    default: return CQ_ERR_UNSUPPORTED;
  }
}

extern "C" int cq_rlayer_matvec_swiglu(const cq_rlayer* L, const void* gate, const void* up, int ld, void* y, int ldy, int M,
                                       uint32_t* status_word, cq_stream_t stream) {
  if (!L || !L->blob || !gate || !up || !y || M < 1) return CQ_ERR_BAD_ARG;
  if (((uintptr_t)gate | (uintptr_t)up | (uintptr_t)y) & 1) return CQ_ERR_BAD_ARG;
  if (ld < L->K || ldy < L->N) return CQ_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  for (int m0 = 0; m0 < M; m0 += RV_MAX_ROWS) {
    const int rows = M - m0 < RV_MAX_ROWS ? M - m0 : RV_MAX_ROWS;
    const __half* gp = (const __half*)gate + (size_t)m0 * ld;
    const __half* up2 = (const __half*)up + (size_t)m0 * ld;
    __half* yp = (__half*)y + (size_t)m0 * ldy;
    int rc = CQ_ERR_UNSUPPORTED;
    switch (rv_gpw_for(L)) {
      case 2: rc = rv_launch(rv_pick<RV_W, 2>(L->bits, L->sets, rows), RV_W, 2, &L, 1, gp, ld, &yp, ldy, rows, 0, status_word, st, nullptr, up2); break;
      case 4: rc = rv_launch(rv_pick<RV_W, 4>(L->bits, L->sets, rows), RV_W, 4, &L, 1, gp, ld, &yp, ldy, rows, 0, status_word, st, nullptr, up2); break;
      default: break;
    }
    if (rc != CQ_OK) return rc;
  }
  return CQ_OK;
}

extern "C" int cq_rlayer_preferred_rows(const cq_rlayer* L) {
  if (!L) return 0;
  const int gpw = rv_gpw_for(L);
  if (!gpw) return 0;
  // measured on B200 through the drop-in ops against the tile GEMM: 8 rows (two launches) take 12 - 16 us
  // against the GEMM's 25 - 33; 16 rows (four launches) 30 / 35 us on 4096 -> 4096 / 11008 against 25 / 32,
  // so three launches are the limit; layers split along K (11008 -> 4096: 14 us per launch) stop at two
  return L->ksplit > 1 ? 8 : 12;
}

extern "C" int cq_rlayer_matvec(const cq_rlayer* L, const void* x, void* y, int accumulate, uint32_t* status_word,
                                cq_stream_t stream) {
  if (!L) return CQ_ERR_BAD_ARG;
  return cq_rlayers_matvec(&L, 1, x, L->K, &y, L->N, 1, accumulate, status_word, stream);
}

namespace {
// x from mapped host memory into device memory: one CTA, 16-byte loads across PCIe.  The dependent matvec
// is released at once, so its weight copies run while these loads are under way.
__global__ void __launch_bounds__(256) rl_copy_in_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int n16,
                                                         const unsigned short* __restrict__ src_tail,
                                                         unsigned short* __restrict__ dst_tail, int ntail) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int i = threadIdx.x; i < n16; i += 256) dst[i] = src[i];
  for (int i = threadIdx.x; i < ntail; i += 256) dst_tail[i] = src_tail[i];
}

// true if the GPU can address this host pointer directly (page-locked, mapped memory)
bool rl_host_mapped(const void* p) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return at.type == cudaMemoryTypeHost && at.devicePointer == p;
}
}  // namespace

extern "C" int cq_rlayer_matvec_host(const cq_rlayer* L, const void* x_host, void* y_host, void* x_dev, void* y_dev,
                                     uint32_t* status_word, cq_stream_t stream) {
  if (!L || !x_host || !y_host || !x_dev || !y_dev) return CQ_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t xb = (size_t)L->K * sizeof(__half), yb = (size_t)L->N * sizeof(__half);
  if (rl_host_mapped(x_host) && rl_host_mapped(y_host) && !((uintptr_t)x_host & 15) && !((uintptr_t)x_dev & 15)) {
    // page-locked buffers: no DMA operations at all.  A one-CTA kernel fetches x across the bus, the matvec
    // (released at once: its weights stream meanwhile) stores y straight into the host buffer.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int n16 = (int)(xb / 16), ntail = (int)((xb - (size_t)n16 * 16) / 2);
    CQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, rl_copy_in_kernel, (const uint4*)x_host, (uint4*)x_dev, n16,
                                   (const unsigned short*)((const uint8_t*)x_host + (size_t)n16 * 16),
                                   (unsigned short*)((uint8_t*)x_dev + (size_t)n16 * 16), ntail));
    const int rc = cq_rlayer_matvec(L, x_dev, y_host, 0, status_word, stream);
    if (rc != CQ_OK) return rc;
    CQ_CUDA_TRY(cudaStreamSynchronize(st));
    return CQ_OK;
  }
  CQ_CUDA_TRY(cudaMemcpyAsync(x_dev, x_host, xb, cudaMemcpyHostToDevice, st));
  const int rc = cq_rlayer_matvec(L, x_dev, y_dev, 0, status_word, stream);
  if (rc != CQ_OK) return rc;
  CQ_CUDA_TRY(cudaMemcpyAsync(y_host, y_dev, yb, cudaMemcpyDeviceToHost, st));
  CQ_CUDA_TRY(cudaStreamSynchronize(st));
  return CQ_OK;
}

