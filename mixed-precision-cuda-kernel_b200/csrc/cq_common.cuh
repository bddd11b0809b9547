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
// Codes inside a granule are stored in the order a warp consumes them with the integer
// tensor-core instruction mma.sync.m16n8k32 (A = 16 rows x 32 k' of unsigned 8-bit codes,
// B = 32 k' x 8 columns of signed 8-bit activations): lane = 4*g + c (g = 0..7, c = 0..3)
// owns rows g and g+8.  MMA m (0..3) covers the granule's columns 32m..32m+31; inside it the
// lane's fragment registers hold, as bytes i = 0..3, the columns
//     kk = 32*m + 16*b + 4*c + i        b = 0: registers a0 (row g), a1 (row g+8)
//                                         b = 1: registers a2 (row g), a3 (row g+8).
// Register j = 2*m + b (0..7) of a row is the unit of packing:
//
//   4-bit: one 32-bit word per (row, m): byte i = code(j = 2m) | code(j = 2m+1) << 4, so
//          `w & 0x0F0F0F0F` and `(w >> 4) & 0x0F0F0F0F` are the two registers.
//          [plane m>>1][lane][16 B] = words {m even: row g, row g+8; m odd: row g, row g+8}.
//   3-bit: three words A, B, C per row; byte i of
//            A = code(j=0) | code(j=1) << 3 | (code(j=6) & 3) << 6
//            B = code(j=2) | code(j=3) << 3 | (code(j=6) >> 2) << 6 | (code(j=7) >> 2) << 7
//            C = code(j=4) | code(j=5) << 3 | (code(j=7) & 3) << 6
//          [lane][16 B] = {A, B, C of row g, A of row g+8}, then at byte 512 [lane][8 B] =
//          {B, C of row g+8}.
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

// ---- stream layout: where code (row rl = 0..15, column kk = 0..127) of a granule sits.
// 4-bit: byte offset of its 32-bit word inside the granule and the shift of the nibble.
__host__ __device__ inline void cq_sl4_pos(int rl, int kk, int* word_off, int* shift) {
  const int m = kk >> 5, b = (kk >> 4) & 1, c = (kk >> 2) & 3, i = kk & 3;
  const int lane = 4 * (rl & 7) + c, r = rl >> 3;
  *word_off = (m >> 1) * 512 + lane * 16 + ((m & 1) * 2 + r) * 4;
  *shift = 8 * i + 4 * b;
}
// 3-bit: byte offset of word w (0 = A, 1 = B, 2 = C) of row rl for the lane that owns column kk.
__host__ __device__ inline int cq_sl3_word_off(int rl, int c, int w) {
  const int lane = 4 * (rl & 7) + c;
  if ((rl >> 3) == 0) return lane * 16 + 4 * w;
  return w == 0 ? lane * 16 + 12 : 512 + lane * 8 + 4 * (w - 1);
}

