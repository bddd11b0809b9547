// GPU re-pack between the reference's buffers (llama/qlinear.py:43-58 of the
// reference project: uint8 qweight (K'/8*bits, N), fp16 scales (NG, N), fp16
// cherry_weight (C, N), int16 cherry_indices (C,)) and the stream layout
// described in cq_common.cuh.  Both directions are pure bit moves, so a
// prepare -> unprepare round trip is byte-identical.
#include "cq_common.cuh"

namespace {

struct LayoutDims {
  int bits, K, N, C, G, Kc, Kp, Cp, n_gran, n_sub, sets, gran_bytes, cher_bytes;
};

LayoutDims dims_of(const cq_layer* L) {
  LayoutDims d;
  d.bits = L->bits; d.K = L->K; d.N = L->N; d.C = L->C; d.G = L->G;
  d.Kc = L->Kc; d.Kp = L->Kp; d.Cp = L->Cp; d.n_gran = L->n_gran; d.n_sub = L->n_sub;
  d.sets = L->sets; d.gran_bytes = L->gran_bytes; d.cher_bytes = L->cher_bytes;
  return d;
}

__device__ __forceinline__ int code_bytes(const LayoutDims& d) { return 256 * d.bits; }

// ---------------------------------------------------------------- prepare: codes
__global__ void prepare_codes_kernel(LayoutDims d, const uint8_t* __restrict__ q,
                                     uint32_t* __restrict__ stream_words) {
  const int wpg = (d.bits == 4) ? 256 : 192;  // 32-bit code words per granule
  const long long total = (long long)d.n_sub * d.n_gran * wpg;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const long long gran = id / wpg;
    const int w = (int)(id % wpg);
    const int sub = (int)(gran / d.n_gran), gi = (int)(gran % d.n_gran);
    uint32_t word = 0;
    int lane, row_local;
    if (d.bits == 4) {
      const int h = w >> 7;
      lane = (w & 127) >> 2;
      const int wq = w & 3;
      row_local = (lane >> 2) + 8 * (wq >> 1);
      const int n = sub * 16 + row_local;
      const int kbase = gi * 128 + h * 64 + 16 * (lane & 3) + 8 * (wq & 1);
      if (n < d.N) {
        for (int i = 0; i < 8; ++i) {
          const int kc = kbase + i;
          if (kc < d.Kc) word |= cq_ref_code(q, 4, kc, n, d.N) << cq_s4_shift(i);
        }
      }
    } else {
      lane = w / 6;
      const int wq = w % 6;
      row_local = (lane >> 2) + 8 * (wq / 3);
      const int wi = wq % 3;
      const int n = sub * 16 + row_local;
      const int kbase = gi * 128 + 16 * (lane & 3);
      if (n < d.N) {
        for (int p = 0; p < 5; ++p) {
          for (int hh = 0; hh < 2; ++hh) {
            const int e = 2 * (5 * wi + p) + hh;
            const int kc = kbase + ((e < 16) ? e : 64 + (e - 16));
            if (kc < d.Kc) word |= cq_ref_code(q, 3, kc, n, d.N) << (16 * hh + 1 + 3 * p);
          }
        }
        for (int hh = 0; hh < 2; ++hh) {  // pair 15: codes e = 30, 31 -> column 64 + 14 + hh
          const int kc = kbase + 64 + 14 + hh;
          if (kc < d.Kc) word |= ((cq_ref_code(q, 3, kc, n, d.N) >> wi) & 1u) << (16 * hh);
        }
      }
    }
    const size_t byte_off = (size_t)gran * d.gran_bytes + (size_t)w * 4;
    stream_words[byte_off >> 2] = word;
  }
}

// ---------------------------------------------------------------- prepare: scales
__global__ void prepare_scales_kernel(LayoutDims d, const __half* __restrict__ scales,
                                      uint8_t* __restrict__ stream) {
  const int per = d.sets * 16;
  const long long total = (long long)d.n_sub * d.n_gran * per;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const long long gran = id / per;
    const int e = (int)(id % per);
    const int sp = e >> 4, r = ((e & 15) >> 1) + 8 * (e & 1);   // [set][g][row g, row g+8]
    const int sub = (int)(gran / d.n_gran), gi = (int)(gran % d.n_gran);
    const int n = sub * 16 + r;
    const int kc0 = gi * 128 + sp * (128 / d.sets);
    __half v = __float2half(0.f);
    if (n < d.N && kc0 < d.Kc) v = scales[(size_t)(kc0 / d.G) * d.N + n];
    __half* dst = reinterpret_cast<__half*>(stream + (size_t)gran * d.gran_bytes + code_bytes(d));
    dst[e] = v;
  }
}

// ---------------------------------------------------------------- prepare: cherries
__global__ void prepare_cherry_kernel(LayoutDims d, const __half* __restrict__ cw,
                                      __half* __restrict__ cstream) {
  const int nj = d.Cp / 16;
  const long long total = (long long)d.n_sub * nj * 32 * 8;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int e = (int)(id & 7);            // half inside the lane's 16 bytes
    const int lane = (int)((id >> 3) & 31);
    const long long blk = id >> 8;          // sub * nj + j
    const int j = (int)(blk % nj), sub = (int)(blk / nj);
    const int g = lane >> 2, t = lane & 3;
    const int reg = e >> 1;                 // a0..a3
    const int c = 16 * j + 2 * t + (e & 1) + 8 * (reg >> 1);
    const int n = sub * 16 + g + 8 * (reg & 1);
    __half v = __float2half(0.f);
    if (c < d.C && n < d.N) v = cw[(size_t)c * d.N + n];
    cstream[id] = v;
  }
}

// ---------------------------------------------------------------- prepare: index maps
// Compact column kc sits at original column kc + shift(kc), shift(kc) = #{m : idx[m] - m <= kc},
// the reference kernel's upper-bound search (csrc/quant_cuda_kernel.cu:785-795).  Stored per
// octet of compact columns: shift of its first column | shift of its last column << 16
// (equal unless a cherry column falls inside the octet); 0xFFFFFFFF past K'.
__global__ void prepare_index_kernel(LayoutDims d, const int16_t* __restrict__ idx,
                                     uint32_t* __restrict__ osh, uint16_t* __restrict__ cidx) {
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

// ---------------------------------------------------------------- stream readers
__device__ __forceinline__ uint32_t stream_code(const LayoutDims& d, const uint8_t* stream, int kc, int n) {
  const int sub = n >> 4, rl = n & 15, g = rl & 7, hi = rl >> 3;
  const int gi = kc >> 7, kk = kc & 127, h = kk >> 6, t = (kk & 63) >> 4, i = kk & 15;
  const int lane = 4 * g + t;
  const uint8_t* gran = stream + ((size_t)sub * d.n_gran + gi) * d.gran_bytes;
  if (d.bits == 4) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(gran + h * 512 + lane * 16 + 4 * (2 * hi + (i >> 3)));
    return (w >> cq_s4_shift(i & 7)) & 0xFu;
  }
  const uint32_t* w = reinterpret_cast<const uint32_t*>(gran + lane * 24 + 12 * hi);
  const int e = 16 * h + i;
  if (e < 30) {
    int word, bit;
    cq_s3_pos(e, &word, &bit);
    return (w[word] >> bit) & 0x7u;
  }
  const int b = 16 * (e & 1);
  return ((w[0] >> b) & 1u) | (((w[1] >> b) & 1u) << 1) | (((w[2] >> b) & 1u) << 2);
}

// ---------------------------------------------------------------- unprepare
__global__ void unprepare_codes_kernel(LayoutDims d, const uint8_t* __restrict__ stream,
                                       uint8_t* __restrict__ q) {
  const long long total = (long long)(d.Kc / 8) * d.N;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(id % d.N);
    const int o = (int)(id / d.N);
    uint32_t word = 0;
    for (int i = 0; i < 8; ++i) word |= stream_code(d, stream, 8 * o + i, n) << (d.bits * i);
    const size_t r = (size_t)o * d.bits;
    for (int b = 0; b < d.bits; ++b) q[(r + b) * d.N + n] = (uint8_t)(word >> (8 * b));
  }
}

__global__ void unprepare_scales_kernel(LayoutDims d, const uint8_t* __restrict__ stream,
                                        __half* __restrict__ scales) {
  const int ng = (d.Kc + d.G - 1) / d.G;
  const long long total = (long long)ng * d.N;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(id % d.N), grp = (int)(id / d.N);
    const int kc0 = grp * d.G;
    const int gi = kc0 >> 7, sp = (kc0 & 127) / (128 / d.sets);
    const uint8_t* gran = stream + ((size_t)(n >> 4) * d.n_gran + gi) * d.gran_bytes;
    scales[id] = reinterpret_cast<const __half*>(gran + code_bytes(d))[sp * 16 + 2 * (n & 7) + ((n >> 3) & 1)];
  }
}

__global__ void unprepare_cherry_kernel(LayoutDims d, const __half* __restrict__ cstream,
                                        const uint16_t* __restrict__ cidx,
                                        __half* __restrict__ cw, int16_t* __restrict__ idx) {
  const long long total = (long long)d.C * d.N;
  const int nj = d.Cp / 16;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(id % d.N), c = (int)(id / d.N);
    const int sub = n >> 4, rl = n & 15, g = rl & 7;
    const int j = c >> 4, cc = c & 15;
    const int t = (cc & 7) >> 1;
    const int reg = (rl >> 3) + 2 * (cc >> 3);
    const int lane = 4 * g + t;
    cw[id] = cstream[(((size_t)sub * nj + j) * 32 + lane) * 8 + 2 * reg + (cc & 1)];
    if (n == 0) idx[c] = (int16_t)cidx[c];
  }
}

int blocks_for(long long total, int threads) {
  long long b = (total + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > 148 * 64) b = 148 * 64;
  return (int)b;
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

}  // namespace

extern "C" int cq_layer_init(cq_layer* L, int bits, int K, int N, int C, int G, void* blob) {
  if (!L) return CQ_ERR_BAD_ARG;
  if (bits != 3 && bits != 4) return CQ_ERR_BAD_BITS;
  if (G == -1) G = K;  // llama/qlinear.py:34
  if (K <= 0 || N <= 0 || C < 0 || K % 8 || N % 8 || C % 8 || C >= K || K > 65534)
    return CQ_ERR_BAD_SHAPE;
  if (!(G == 64 || (G > 0 && G % 128 == 0))) return CQ_ERR_BAD_GROUP;
  if (blob && ((uintptr_t)blob & 255)) return CQ_ERR_BAD_ARG;
  L->bits = bits; L->K = K; L->N = N; L->C = C; L->G = G;
  L->Kc = K - C;
  L->n_gran = (L->Kc + 127) / 128;
  L->Kp = L->n_gran * 128;
  L->Cp = (C + 15) / 16 * 16;
  L->n_sub = (N + 15) / 16;
  L->sets = (G == 64) ? 2 : 1;
  L->gran_bytes = 256 * bits + L->sets * 32;
  L->cher_bytes = (L->Cp / 16) * 512;
  size_t off = 0;
  L->off_stream = off; off = align256(off + (size_t)L->n_sub * L->n_gran * L->gran_bytes);
  L->off_cherry = off; off = align256(off + (size_t)L->n_sub * L->cher_bytes);
  L->off_osh = off;    off = align256(off + (size_t)(L->Kp / 8) * 4);
  L->off_cidx = off;   off = align256(off + (size_t)(L->Cp ? L->Cp : 16) * 2);
  L->blob_bytes = off;
  L->blob = blob;
  return CQ_OK;
}

extern "C" int cq_layer_prepare(const cq_layer* L, const uint8_t* qweight, const void* scales,
                                const void* cherry_weight, const int16_t* cherry_indices,
                                cq_stream_t stream_) {
  if (!L || !L->blob || !qweight || !scales) return CQ_ERR_BAD_ARG;
  if (L->C > 0 && (!cherry_weight || !cherry_indices)) return CQ_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream_;
  const LayoutDims d = dims_of(L);
  uint8_t* blob = (uint8_t*)L->blob;
  const int T = 256;
  const long long words = (long long)d.n_sub * d.n_gran * (d.bits == 4 ? 256 : 192);
  prepare_codes_kernel<<<blocks_for(words, T), T, 0, st>>>(d, qweight, (uint32_t*)(blob + L->off_stream));
  prepare_scales_kernel<<<blocks_for((long long)d.n_sub * d.n_gran * d.sets * 16, T), T, 0, st>>>(
      d, (const __half*)scales, blob + L->off_stream);
  if (d.Cp > 0)
    prepare_cherry_kernel<<<blocks_for((long long)d.n_sub * (d.Cp / 16) * 256, T), T, 0, st>>>(
        d, (const __half*)cherry_weight, (__half*)(blob + L->off_cherry));
  const int m = d.Kp / 8 > d.Cp ? d.Kp / 8 : d.Cp;
  prepare_index_kernel<<<(m + T - 1) / T, T, 0, st>>>(d, cherry_indices, (uint32_t*)(blob + L->off_osh),
                                                      (uint16_t*)(blob + L->off_cidx));
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}

extern "C" int cq_layer_unprepare(const cq_layer* L, uint8_t* qweight, void* scales,
                                  void* cherry_weight, int16_t* cherry_indices, cq_stream_t stream_) {
  if (!L || !L->blob || !qweight || !scales) return CQ_ERR_BAD_ARG;
  if (L->C > 0 && (!cherry_weight || !cherry_indices)) return CQ_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream_;
  const LayoutDims d = dims_of(L);
  const uint8_t* blob = (const uint8_t*)L->blob;
  const int T = 256;
  unprepare_codes_kernel<<<blocks_for((long long)(d.Kc / 8) * d.N, T), T, 0, st>>>(d, blob + L->off_stream, qweight);
  const int ng = (d.Kc + d.G - 1) / d.G;
  unprepare_scales_kernel<<<blocks_for((long long)ng * d.N, T), T, 0, st>>>(d, blob + L->off_stream, (__half*)scales);
  if (d.C > 0)
    unprepare_cherry_kernel<<<blocks_for((long long)d.C * d.N, T), T, 0, st>>>(
        d, (const __half*)(blob + L->off_cherry), (const uint16_t*)(blob + L->off_cidx),
        (__half*)cherry_weight, cherry_indices);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}
