// fp32-I/O variant of the 3-bit operator, selected by `fp16 == false` in the
// reference (csrc/quant_cuda_kernel.cu:159-179 of the reference project:
// VecQuant3MatMulKernelCherryQBatched / ...G64, float x / scales / cherry / mul,
// int32 indices).  Only the reference's micro-benchmark uses it
// (benchmark_speed.py:32).  It reads the reference's uint8 layout directly and
// keeps the reference's arithmetic — fp32 products, scale applied to the sum
// over each group, fp32 atomicAdd into `mul` — with two fixes: the activation
// slice is re-staged behind barriers for every batch tile, and threads past the
// last column stay in the barriers instead of returning early.
#include "cq_common.cuh"

namespace {

constexpr int TILE_M = 16;

template <int BITS>
__global__ void __launch_bounds__(128) matvec_f32_kernel(
    const float* __restrict__ x, const uint8_t* __restrict__ q, const float* __restrict__ cw,
    const int32_t* __restrict__ idx, const float* __restrict__ sf, float* __restrict__ mul,
    int M, int K, int N, int C, int G) {
  __shared__ float xs[TILE_M][128];
  const int Kc = K - C;
  const int nslice = (Kc + 127) / 128;
  const int tid = threadIdx.x;
  const int col = 128 * blockIdx.y + tid;
  const bool cherry_block = (int)blockIdx.x >= nslice;
  const float off = (float)(1 << (BITS - 1)) - 0.5f;

  // original column this thread stages
  int src = -1;
  if (!cherry_block) {
    const int kc = 128 * blockIdx.x + tid;
    if (kc < Kc) {
      int low = 0, high = C;
      while (low < high) {
        const int mid = (low + high) >> 1;
        if (idx[mid] - mid <= kc) low = mid + 1; else high = mid;
      }
      src = kc + low;
    }
  } else {
    const int c = 128 * ((int)blockIdx.x - nslice) + tid;
    if (c < C) src = idx[c];
  }

  for (int m0 = 0; m0 < M; m0 += TILE_M) {
    const int mt = min(TILE_M, M - m0);
    __syncthreads();
    for (int m = 0; m < mt; ++m) xs[m][tid] = (src >= 0) ? x[(size_t)(m0 + m) * K + src] : 0.f;
    __syncthreads();
    if (col >= N) continue;
    float acc[TILE_M];
#pragma unroll
    for (int m = 0; m < TILE_M; ++m) acc[m] = 0.f;
    if (cherry_block) {
      const int c0 = 128 * ((int)blockIdx.x - nslice);
      const int len = min(128, C - c0);
      for (int i = 0; i < len; ++i) {
        const float wv = cw[(size_t)(c0 + i) * N + col];
#pragma unroll
        for (int m = 0; m < TILE_M; ++m)
          if (m < mt) acc[m] += wv * xs[m][i];
      }
    } else {
      const int k0 = 128 * blockIdx.x;
      const int len = min(128, Kc - k0);
      for (int j = 0; j < len; j += 8) {
        const size_t r = (size_t)((k0 + j) >> 3) * BITS;
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < BITS; ++b) word |= (uint32_t)__ldg(q + (r + b) * N + col) << (8 * b);
        const float s = sf[(size_t)((k0 + j) / G) * N + col];
        float wv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) wv[i] = (float)((word >> (BITS * i)) & ((1u << BITS) - 1)) - off;
#pragma unroll
        for (int m = 0; m < TILE_M; ++m) {
          if (m < mt) {
            float part = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) part += wv[i] * xs[m][j + i];
            acc[m] += s * part;
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < TILE_M; ++m)
      if (m < mt) atomicAdd(mul + (size_t)(m0 + m) * N + col, acc[m]);
  }
}

}  // namespace

// Host launcher used by cq_vecquant3matmul_cherryq (fp16 == 0).
int cq_launch_matvec_f32(int bits, const float* x, const uint8_t* q, const float* cw, const int32_t* idx,
                         const float* sf, float* mul, int M, int K, int N, int C, int G, cudaStream_t st) {
  const int Kc = K - C;
  dim3 grid((Kc + 127) / 128 + (C + 127) / 128, (N + 127) / 128), block(128);
  if (bits == 3)
    matvec_f32_kernel<3><<<grid, block, 0, st>>>(x, q, cw, idx, sf, mul, M, K, N, C, G);
  else
    matvec_f32_kernel<4><<<grid, block, 0, st>>>(x, q, cw, idx, sf, mul, M, K, N, C, G);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}
