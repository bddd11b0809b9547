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
    // which (lane, row half r, word) this 32-bit word is: the inverse of cq_sl4_pos / cq_sl3_word_off
    if (d.bits == 4) {
      const int plane = w >> 7, lane = (w & 127) >> 2, wq = w & 3;
      const int m = 2 * plane + (wq >> 1), r = wq & 1;
      const int n = sub * 16 + (lane >> 2) + 8 * r, c = lane & 3;
      if (n < d.N) {
        for (int b = 0; b < 2; ++b)
          for (int i = 0; i < 4; ++i) {
            const int kc = gi * 128 + 32 * m + 16 * b + 4 * c + i;
            if (kc < d.Kc) word |= cq_ref_code(q, 4, kc, n, d.N) << (8 * i + 4 * b);
          }
      }
    } else {
      int lane, r, wi;
      if (w < 128) {
        lane = w >> 2;
        r = ((w & 3) == 3) ? 1 : 0;
        wi = r ? 0 : (w & 3);
      } else {
        lane = (w - 128) >> 1;
        r = 1;
        wi = 1 + ((w - 128) & 1);
      }
      const int n = sub * 16 + (lane >> 2) + 8 * r, c = lane & 3;
      if (n < d.N) {
        // code of fragment register j (0..7), byte i
        auto code = [&](int j, int i) -> uint32_t {
          const int kc = gi * 128 + 32 * (j >> 1) + 16 * (j & 1) + 4 * c + i;
          return kc < d.Kc ? cq_ref_code(q, 3, kc, n, d.N) : 0u;
        };
        for (int i = 0; i < 4; ++i) {
          uint32_t byte;
          if (wi == 0) byte = code(0, i) | (code(1, i) << 3) | ((code(6, i) & 3u) << 6);
          else if (wi == 1) byte = code(2, i) | (code(3, i) << 3) | ((code(6, i) >> 2) << 6) | ((code(7, i) >> 2) << 7);
          else byte = code(4, i) | (code(5, i) << 3) | ((code(7, i) & 3u) << 6);
          word |= byte << (8 * i);
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
  const int sub = n >> 4, rl = n & 15;
  const int gi = kc >> 7, kk = kc & 127;
  const uint8_t* gran = stream + ((size_t)sub * d.n_gran + gi) * d.gran_bytes;
  if (d.bits == 4) {
    int off, shift;
    cq_sl4_pos(rl, kk, &off, &shift);
    return (*reinterpret_cast<const uint32_t*>(gran + off) >> shift) & 0xFu;
  }
  const int j = 2 * (kk >> 5) + ((kk >> 4) & 1), c = (kk >> 2) & 3, i = kk & 3;
  auto byte_of = [&](int w) -> uint32_t {
    return (*reinterpret_cast<const uint32_t*>(gran + cq_sl3_word_off(rl, c, w)) >> (8 * i)) & 0xFFu;
  };
  if (j < 6) return (byte_of(j >> 1) >> (3 * (j & 1))) & 0x7u;
  if (j == 6) return (byte_of(0) >> 6) | (((byte_of(1) >> 6) & 1u) << 2);
  return (byte_of(2) >> 6) | ((byte_of(1) >> 7) << 2);
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
