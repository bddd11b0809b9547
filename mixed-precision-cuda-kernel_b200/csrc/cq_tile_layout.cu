// GPU re-pack between the reference's buffers (llama/qlinear.py:43-58 of the reference
// project) and the tile layout of the tcgen05 kernels (cq_tile.cuh).  Pure bit moves in both
// directions: prepare -> unprepare is byte-identical.
#include "cq_tile.cuh"

namespace {

__device__ __forceinline__ size_t gran_off(const TileDims& d, int tile, int g) {
  return (size_t)tile * d.tile_bytes + (size_t)d.n_cher * CQT_CHER_BYTES + (size_t)g * d.gran_bytes;
}

// One thread per 32-bit code word of the stream.
__global__ void tprepare_codes_kernel(TileDims d, const uint8_t* __restrict__ q, uint8_t* __restrict__ stream) {
  const int wpr = 4 * d.bits;                      // words per row per granule
  const long long total = (long long)d.n_tile * d.n_gran * CQT_ROWS * wpr;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    // id = ((tile * n_gran + g) * bits + chunk) * 128 * 4 + row * 4 + e   (the memory order)
    const int e = (int)(id & 3);
    const int row = (int)((id >> 2) & 127);
    long long rest = id >> 9;
    const int chunk = (int)(rest % d.bits);
    rest /= d.bits;
    const int g = (int)(rest % d.n_gran), tile = (int)(rest / d.n_gran);
    const int wi = 4 * chunk + e;
    const int n = tile * CQT_ROWS + row;
    uint32_t word = 0;
    if (n < d.N) {
      if (d.bits == 4) {
        const int k0 = g * 128 + 8 * wi;
        for (int j = 0; j < 8; ++j)
          if (k0 + j < d.Kc) word |= cq_ref_code(q, 4, k0 + j, n, d.N) << cq_s4_shift(j);
      } else {
        const int t = wi / 3, wq = wi % 3;
        const int k0 = g * 128 + 32 * t;
        for (int p = 0; p < 5; ++p)
          for (int hh = 0; hh < 2; ++hh) {
            const int kc = k0 + 2 * (5 * wq + p) + hh;
            if (kc < d.Kc) word |= cq_ref_code(q, 3, kc, n, d.N) << (16 * hh + 1 + 3 * p);
          }
        for (int hh = 0; hh < 2; ++hh) {
          const int kc = k0 + 30 + hh;
          if (kc < d.Kc) word |= ((cq_ref_code(q, 3, kc, n, d.N) >> wq) & 1u) << (16 * hh);
        }
      }
    }
    uint32_t* dst = reinterpret_cast<uint32_t*>(stream + gran_off(d, tile, g) + (size_t)chunk * 2048 + row * 16 + e * 4);
    *dst = word;
  }
}

__global__ void tprepare_scales_kernel(TileDims d, const __half* __restrict__ scales, uint8_t* __restrict__ stream) {
  const long long total = (long long)d.n_tile * d.n_gran * d.sets * CQT_ROWS;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(id & 127);
    long long rest = id >> 7;
    const int sp = (int)(rest % d.sets);
    rest /= d.sets;
    const int g = (int)(rest % d.n_gran), tile = (int)(rest / d.n_gran);
    const int n = tile * CQT_ROWS + row;
    const int kc0 = g * 128 + sp * (128 / d.sets);
    __half v = __float2half(0.f);
    if (n < d.N && kc0 < d.Kc) v = scales[(size_t)(kc0 / d.G) * d.N + n];
    reinterpret_cast<__half*>(stream + gran_off(d, tile, g) + 2048 * d.bits)[sp * CQT_ROWS + row] = v;
  }
}

__global__ void tprepare_cherry_kernel(TileDims d, const __half* __restrict__ cw, uint8_t* __restrict__ stream) {
  const long long total = (long long)d.n_tile * d.n_cher * 2 * CQT_ROWS * 8;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int e = (int)(id & 7);
    const int row = (int)((id >> 3) & 127);
    const int qq = (int)((id >> 10) & 1);
    const long long rest = id >> 11;
    const int j = (int)(rest % d.n_cher), tile = (int)(rest / d.n_cher);
    const int c = 16 * j + 8 * qq + e, n = tile * CQT_ROWS + row;
    __half v = __float2half(0.f);
    if (c < d.C && n < d.N) v = cw[(size_t)c * d.N + n];
    reinterpret_cast<__half*>(stream + (size_t)tile * d.tile_bytes + (size_t)j * CQT_CHER_BYTES)[(qq * CQT_ROWS + row) * 8 + e] = v;
  }
}

// Same index maps as the stream layout (see cq_layout.cu).
__global__ void tprepare_index_kernel(TileDims d, const int16_t* __restrict__ idx, uint32_t* __restrict__ osh,
                                      uint16_t* __restrict__ cidx) {
  const int id = blockIdx.x * blockDim.x + threadIdx.x;
  if (id < d.Kp / 8) {
    uint32_t v = 0xFFFFFFFFu;
    const int k0 = 8 * id;
    if (k0 < d.Kc) {
      int sh[2];
      for (int e = 0; e < 2; ++e) {
        const int k = k0 + 7 * e;
        int low = 0, high = d.C;
        while (low < high) {
          const int mid = (low + high) >> 1;
          if ((int)idx[mid] - mid <= k) low = mid + 1; else high = mid;
        }
        sh[e] = low;
      }
      v = (uint32_t)sh[0] | ((uint32_t)sh[1] << 16);
    }
    osh[id] = v;
  }
  if (id < d.Cp) cidx[id] = (id < d.C) ? (uint16_t)idx[id] : (uint16_t)CQ_PAD_COL;
}

__device__ __forceinline__ uint32_t tile_code(const TileDims& d, const uint8_t* stream, int kc, int n) {
  const int tile = n >> 7, row = n & 127, g = kc >> 7, kk = kc & 127;
  const uint8_t* gran = stream + gran_off(d, tile, g);
  if (d.bits == 4) {
    const int wi = kk >> 3;
    const uint32_t w = *reinterpret_cast<const uint32_t*>(gran + (wi >> 2) * 2048 + row * 16 + (wi & 3) * 4);
    return (w >> cq_s4_shift(kk & 7)) & 0xFu;
  }
  const int t = kk >> 5, e = kk & 31;
  uint32_t w[3];
  for (int i = 0; i < 3; ++i) {
    const int wi = 3 * t + i;
    w[i] = *reinterpret_cast<const uint32_t*>(gran + (wi >> 2) * 2048 + row * 16 + (wi & 3) * 4);
  }
  if (e < 30) {
    const int qp = e >> 1;
    return (w[qp / 5] >> (16 * (e & 1) + 1 + 3 * (qp % 5))) & 0x7u;
  }
  const int b = 16 * (e & 1);
  return ((w[0] >> b) & 1u) | (((w[1] >> b) & 1u) << 1) | (((w[2] >> b) & 1u) << 2);
}

__global__ void tunprepare_codes_kernel(TileDims d, const uint8_t* __restrict__ stream, uint8_t* __restrict__ q) {
  const long long total = (long long)(d.Kc / 8) * d.N;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(id % d.N), o = (int)(id / d.N);
    uint32_t word = 0;
    for (int i = 0; i < 8; ++i) word |= tile_code(d, stream, 8 * o + i, n) << (d.bits * i);
    const size_t r = (size_t)o * d.bits;
    for (int b = 0; b < d.bits; ++b) q[(r + b) * d.N + n] = (uint8_t)(word >> (8 * b));
  }
}

__global__ void tunprepare_scales_kernel(TileDims d, const uint8_t* __restrict__ stream, __half* __restrict__ scales) {
  const int ng = (d.Kc + d.G - 1) / d.G;
  const long long total = (long long)ng * d.N;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(id % d.N), grp = (int)(id / d.N);
    const int kc0 = grp * d.G;
    const int g = kc0 >> 7, sp = (kc0 & 127) / (128 / d.sets);
    scales[id] = reinterpret_cast<const __half*>(stream + gran_off(d, n >> 7, g) + 2048 * d.bits)[sp * CQT_ROWS + (n & 127)];
  }
}

__global__ void tunprepare_cherry_kernel(TileDims d, const uint8_t* __restrict__ stream,
                                         const uint16_t* __restrict__ cidx, __half* __restrict__ cw,
                                         int16_t* __restrict__ idx) {
  const long long total = (long long)d.C * d.N;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(id % d.N), c = (int)(id / d.N);
    const int j = c >> 4, qq = (c >> 3) & 1, e = c & 7;
    cw[id] = reinterpret_cast<const __half*>(stream + (size_t)(n >> 7) * d.tile_bytes + (size_t)j * CQT_CHER_BYTES)[(qq * CQT_ROWS + (n & 127)) * 8 + e];
    if (n == 0) idx[c] = (int16_t)cidx[c];
  }
}

int tblocks(long long total, int threads) {
  long long b = (total + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > 148 * 64) b = 148 * 64;
  return (int)b;
}

size_t talign256(size_t x) { return (x + 255) & ~(size_t)255; }

}  // namespace

extern "C" int cq_tlayer_init(cq_tlayer* L, int bits, int K, int N, int C, int G, void* blob) {
  if (!L) return CQ_ERR_BAD_ARG;
  if (bits != 3 && bits != 4) return CQ_ERR_BAD_BITS;
  if (G == -1) G = K;
  if (K <= 0 || N <= 0 || C < 0 || K % 8 || N % 8 || C % 8 || C >= K || K > 65534) return CQ_ERR_BAD_SHAPE;
  if (!(G == 64 || (G > 0 && G % 128 == 0))) return CQ_ERR_BAD_GROUP;
  if (blob && ((uintptr_t)blob & 255)) return CQ_ERR_BAD_ARG;
  L->bits = bits; L->K = K; L->N = N; L->C = C; L->G = G;
  L->Kc = K - C;
  L->n_gran = (L->Kc + 127) / 128;
  L->Kp = L->n_gran * 128;
  L->Cp = (C + 15) / 16 * 16;
  L->n_tile = (N + CQT_ROWS - 1) / CQT_ROWS;
  L->n_cher = L->Cp / 16;
  L->sets = (G == 64) ? 2 : 1;
  L->gran_bytes = 2048 * bits + 256 * L->sets;
  L->tile_bytes = L->n_cher * CQT_CHER_BYTES + L->n_gran * L->gran_bytes;
  size_t off = 0;
  L->off_stream = off; off = talign256(off + (size_t)L->n_tile * L->tile_bytes);
  L->off_cidx = off;   off = talign256(off + (size_t)(L->Cp ? L->Cp : 16) * 2);
  L->off_osh = off;    off = talign256(off + (size_t)(L->Kp / 8) * 4);
  L->blob_bytes = off;
  L->blob = blob;
  return CQ_OK;
}

extern "C" int cq_tlayer_prepare(const cq_tlayer* L, const uint8_t* qweight, const void* scales,
                                 const void* cherry_weight, const int16_t* cherry_indices, cq_stream_t stream_) {
  if (!L || !L->blob || !qweight || !scales) return CQ_ERR_BAD_ARG;
  if (L->C > 0 && (!cherry_weight || !cherry_indices)) return CQ_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream_;
  const TileDims d = tile_dims_of(L);
  uint8_t* blob = (uint8_t*)L->blob;
  const int T = 256;
  tprepare_codes_kernel<<<tblocks((long long)d.n_tile * d.n_gran * CQT_ROWS * 4 * d.bits, T), T, 0, st>>>(
      d, qweight, blob + L->off_stream);
  tprepare_scales_kernel<<<tblocks((long long)d.n_tile * d.n_gran * d.sets * CQT_ROWS, T), T, 0, st>>>(
      d, (const __half*)scales, blob + L->off_stream);
  if (d.n_cher > 0)
    tprepare_cherry_kernel<<<tblocks((long long)d.n_tile * d.n_cher * 2048, T), T, 0, st>>>(
        d, (const __half*)cherry_weight, blob + L->off_stream);
  const int m = d.Kp / 8 > d.Cp ? d.Kp / 8 : d.Cp;
  tprepare_index_kernel<<<(m + T - 1) / T, T, 0, st>>>(d, cherry_indices, (uint32_t*)(blob + L->off_osh),
                                                       (uint16_t*)(blob + L->off_cidx));
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}

extern "C" int cq_tlayer_unprepare(const cq_tlayer* L, uint8_t* qweight, void* scales, void* cherry_weight,
                                   int16_t* cherry_indices, cq_stream_t stream_) {
  if (!L || !L->blob || !qweight || !scales) return CQ_ERR_BAD_ARG;
  if (L->C > 0 && (!cherry_weight || !cherry_indices)) return CQ_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream_;
  const TileDims d = tile_dims_of(L);
  const uint8_t* blob = (const uint8_t*)L->blob;
  const int T = 256;
  tunprepare_codes_kernel<<<tblocks((long long)(d.Kc / 8) * d.N, T), T, 0, st>>>(d, blob + L->off_stream, qweight);
  const int ng = (d.Kc + d.G - 1) / d.G;
  tunprepare_scales_kernel<<<tblocks((long long)ng * d.N, T), T, 0, st>>>(d, blob + L->off_stream, (__half*)scales);
  if (d.C > 0)
    tunprepare_cherry_kernel<<<tblocks((long long)d.C * d.N, T), T, 0, st>>>(
        d, blob + L->off_stream, (const uint16_t*)(blob + L->off_cidx), (__half*)cherry_weight, cherry_indices);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}
