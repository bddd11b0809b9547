// Tile layout of a prepared CherryQ layer for the tcgen05 (UMMA) kernels.
//
//   row tile   = 128 consecutive output rows n (one TMEM lane each)
//   granule    = one row tile x 128 consecutive COMPACT columns k'
//   cherry item= one row tile x 16 consecutive cherry columns (fp16)
//   stream     = n_tile blocks of `tile_bytes`, each
//                  [n_cher cherry items of 4096 B][n_gran granules of gran_bytes]
//
// Cherry item j : [q = 0,1][row 0..127][8 fp16] = cherry_weight[16j + 8q + e][n]
// Granule       : [q = 0..bits-1][row 0..127][16 B] codes, then [set][row] fp16 scales.
//   A row's words w_i (i = 4q + e) hold its 128 codes in the order the kernel needs to
//   write them to tensor memory as K-major fp16 pairs (column c = k'/2 holds k' = 2c, 2c+1):
//   4-bit: w_i holds k' = 8i..8i+7; code j of the word sits at nibble (j>>1) + 4*(j&1), so
//          one AND yields the pair (2p, 2p+1) in the (low, high) halves of a register.
//   3-bit: words 3t..3t+2 hold k' = 32t..32t+31; pair q = 0..14 (codes 2q, 2q+1) sits in word
//          3t + q/5 at bits 16*(code&1) + 1 + 3*(q%5); pair 15 is spread over bit 16*(code&1)
//          of the three words (code bit 0, 1, 2).
//
//   cidx  = Cp uint16 sorted cherry columns (0xFFFF past C)
//   osh   = Kp/8 uint32 per octet of compact columns: shift of first | last << 16, ~0 past K'
#pragma once

#include "cq_common.cuh"

#define CQT_ROWS 128
#define CQT_CHER_BYTES 4096

struct TileDims {
  int bits, K, N, C, G, Kc, Kp, Cp, n_gran, n_tile, n_cher, sets, gran_bytes, tile_bytes;
};

__host__ __device__ inline TileDims tile_dims_of(const cq_tlayer* L) {
  TileDims d;
  d.bits = L->bits; d.K = L->K; d.N = L->N; d.C = L->C; d.G = L->G;
  d.Kc = L->Kc; d.Kp = L->Kp; d.Cp = L->Cp; d.n_gran = L->n_gran; d.n_tile = L->n_tile;
  d.n_cher = L->n_cher; d.sets = L->sets; d.gran_bytes = L->gran_bytes; d.tile_bytes = L->tile_bytes;
  return d;
}
