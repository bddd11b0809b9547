// Shared definitions of the CherryQ B200 library: the stream layout that the
// re-pack kernels write and the matvec kernels read, and small helpers.
//
// Stream layout of one prepared layer (all sizes in bytes, little endian):
//
//   sub-tile  = 16 consecutive output rows n
//   granule   = one sub-tile x 128 consecutive COMPACT columns k' (cherry columns
//               removed, original order kept) — the unit of work distribution
//   stream    = n_sub x n_gran granules, sub-tile major, each `gran_bytes` long:
//                 [codes: 16 rows x 128 codes x bits/8][scales: sets x 8 x (row g, row g+8) fp16]
//
// Codes inside a granule are stored in the order a warp consumes them with
// mma.sync.m16n8k16 (A = 16 rows x 16 k' of weights, B = 16 k' x 8 batch):
// lane = 4*g + t (g = 0..7, t = 0..3) owns rows g and g+8 and, in each 64-column
// half `h` of the granule, the 16 compact columns k' = 128*gran + 64*h + 16*t + i.
// MMA m (0..3) of a half uses the lane's columns i = 4m..4m+3, as fragment
// registers a0/a1 (i = 4m, 4m+1; rows g / g+8) and a2/a3 (i = 4m+2, 4m+3).
//
//   4-bit: [half h][lane][16 B] = words {row g: i=0..7, i=8..15, row g+8: i=0..7, i=8..15};
//          inside a word code i sits at nibble (i>>1) + 4*(i&1), so that one mask
//          yields the fp16 pair (i, i+1) in the (low, high) halves of a register.
//   3-bit: [lane][24 B] = words {row g: w0 w1 w2, row g+8: w0 w1 w2}; a row's 32
//          codes e (e<16: half 0, i=e; e>=16: half 1, i=e-16) form pairs q = e>>1;
//          pair q < 15 lives in word q/5 at bit 16*(e&1) + 1 + 3*(q%5); pair 15
//          (e = 30, 31) is spread over bit 16*(e&1) of w0 (code bit 0), w1 (bit 1),
//          w2 (bit 2).
//
//   cherry stream = n_sub blocks of (Cp/16) x [lane][16 B] fp16 A-fragments:
//          a0 = W[c=16j+2t, 2t+1][row g], a1 = same c, row g+8, a2/a3 = c + 8.
//   osh   = Kp/8 uint32: per octet of compact columns, how far its first | last << 16 column is
//          shifted in the original row (number of cherry columns before it); ~0 past K'.
//   cidx  = Cp uint16: sorted cherry columns (0xFFFF past C).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cherryq.h"

#define CQ_ROWS_PER_SUB 16
#define CQ_GRAN_K 128
#define CQ_PAD_COL 0xFFFFu

// thread-local record of the last CUDA error (defined in cq_api.cu)
void cq_set_cuda_error(int err);

#define CQ_CUDA_TRY(expr)                       \
  do {                                          \
    cudaError_t _e = (expr);                    \
    if (_e != cudaSuccess) {                    \
      cq_set_cuda_error((int)_e);               \
      (void)cudaGetLastError();                 \
      return CQ_ERR_CUDA;                       \
    }                                           \
  } while (0)

// Unsigned code u of (compact column kc, row n) in the reference's uint8 layout
// (qweight (K'/8*bits, N), N contiguous).
//   4-bit: byte kc>>1, low nibble first.
//   3-bit: 8 codes = little-endian 24-bit word over 3 consecutive byte rows.
__host__ __device__ inline uint32_t cq_ref_code(const uint8_t* q, int bits, int kc, int n, int N) {
  if (bits == 4) {
    uint32_t b = q[(size_t)(kc >> 1) * N + n];
    return (b >> (4 * (kc & 1))) & 0xFu;
  }
  size_t r = (size_t)(kc >> 3) * 3;
  uint32_t w = (uint32_t)q[r * N + n] | ((uint32_t)q[(r + 1) * N + n] << 8) |
               ((uint32_t)q[(r + 2) * N + n] << 16);
  return (w >> (3 * (kc & 7))) & 0x7u;
}

// Position of a 4-bit code inside its 32-bit stream word: i = 0..7.
__host__ __device__ inline int cq_s4_shift(int i) { return 4 * ((i >> 1) + 4 * (i & 1)); }

// Position of 3-bit code e (0..29) of a row inside words w0..w2: word and bit.
__host__ __device__ inline void cq_s3_pos(int e, int* word, int* bit) {
  int q = e >> 1;
  *word = q / 5;
  *bit = 16 * (e & 1) + 1 + 3 * (q % 5);
}
