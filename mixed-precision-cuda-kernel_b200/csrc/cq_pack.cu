// GPU versions of the reference's host-side layer conversion code
// (paths inside the reference project):
//   llama/qlinear.py:67-118   QuantLinear.pack    -> cq_pack
//   llama/qlinear.py:120-162  QuantLinear.unpack  -> cq_unpack_dense
//   csrc/quant_cuda_kernel.cu:838-1010 Dequantize{3,4}Normal -> cq_dequantize{3,4}_normal
// All three are bit-exact with the reference's torch arithmetic: fp16 element-wise
// operations are evaluated in fp32 and rounded once to fp16, exactly as torch does.
#include "cq_common.cuh"

namespace {

// number of sorted cherry columns with idx[m] - m <= kc (compact -> original shift)
__device__ __forceinline__ int cherry_shift(const int16_t* __restrict__ idx, int C, int kc) {
  int low = 0, high = C;
  while (low < high) {
    const int mid = (low + high) >> 1;
    if ((int)idx[mid] - mid <= kc) low = mid + 1; else high = mid;
  }
  return low;
}

__device__ __forceinline__ float load_w(const void* w, int is_f32, size_t i) {
  return is_f32 ? reinterpret_cast<const float*>(w)[i]
                : __half2float(reinterpret_cast<const __half*>(w)[i]);
}

// ------------------------------------------------------------------ pack
// llama/qlinear.py:72 — sort the cherry columns (rank sort; they are distinct).
__global__ void pack_sort_kernel(const int32_t* __restrict__ in, int C, int16_t* __restrict__ out) {
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < C; c += gridDim.x * blockDim.x) {
    const int v = in[c];
    int rank = 0;
    for (int m = 0; m < C; ++m) rank += (in[m] < v) || (in[m] == v && m < c);
    out[rank] = (int16_t)v;
  }
}

// llama/qlinear.py:74 — cherry_weight[c, n] = fp16(W[n, idx[c]]).
__global__ void pack_cherry_kernel(const void* __restrict__ w, int is_f32, const int16_t* __restrict__ idx,
                                   int K, int N, int C, __half* __restrict__ cw) {
  const long long total = (long long)C * N;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(id % N), c = (int)(id / N);
    cw[id] = __float2half_rn(load_w(w, is_f32, (size_t)n * K + idx[c]));
  }
}

// llama/cherry_linear.py:69-75 + llama/quantizer.py:148-152 + llama/qlinear.py:78:
// s = fp16((max|w| + 1e-6) / 2^(bits-1)) per (row, group of the compact axis), evaluated in
// the weight dtype.  One warp per (n, group).
__global__ void pack_scales_kernel(const void* __restrict__ w, int is_f32, const int16_t* __restrict__ idx,
                                   int bits, int K, int N, int C, int G, __half* __restrict__ scales) {
  const int Kc = K - C, ng = (Kc + G - 1) / G;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long id = warp0; id < (long long)ng * N; id += nwarps) {
    const int grp = (int)(id % ng), n = (int)(id / ng);
    const int k0 = grp * G, k1 = min(Kc, k0 + G);
    float mx = 0.f;
    for (int kc = k0 + lane; kc < k1; kc += 32)
      mx = fmaxf(mx, fabsf(load_w(w, is_f32, (size_t)n * K + kc + cherry_shift(idx, C, kc))));
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) {
      const float div = (float)(1 << (bits - 1));
      __half s;
      if (is_f32) {
        s = __float2half_rn(__fdiv_rn(__fadd_rn(mx, 1e-6f), div));
      } else {
        const __half a = __float2half_rn(__fadd_rn(mx, 1e-6f));   // fp16 add, rounded once
        s = __float2half_rn(__fdiv_rn(__half2float(a), div));     // fp16 divide, rounded once
      }
      scales[(size_t)grp * N + n] = s;
    }
  }
}

// llama/quantizer.py:154-158 + llama/qlinear.py:81-116: quantize 8 compact columns of one
// row and write their 3 or 4 bytes.
__global__ void pack_codes_kernel(const void* __restrict__ w, int is_f32, const int16_t* __restrict__ idx,
                                  const __half* __restrict__ scales, int bits, int K, int N, int C,
                                  int G, uint8_t* __restrict__ q) {
  const int Kc = K - C;
  const long long total = (long long)(Kc / 8) * N;
  const float qmax = (float)((double)(1 << (bits - 1)) - 1e-2);
  const int qoff = 1 << (bits - 1);
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(id % N), o = (int)(id / N);
    uint32_t word = 0;
    for (int i = 0; i < 8; ++i) {
      const int kc = 8 * o + i;
      const float wv = load_w(w, is_f32, (size_t)n * K + kc + cherry_shift(idx, C, kc));
      const float s = __half2float(scales[(size_t)(kc / G) * N + n]);
      float r = __fdiv_rn(wv, s);
      if (!is_f32) r = __half2float(__float2half_rn(r));  // fp16 / fp16 is rounded to fp16
      r = fminf(fmaxf(r, -qmax), qmax);
      const int code = (int)rintf(__fsub_rn(r, 0.5f)) + qoff;
      word |= (uint32_t)(code & ((1 << bits) - 1)) << (bits * i);
    }
    for (int b = 0; b < bits; ++b) q[((size_t)o * bits + b) * N + n] = (uint8_t)(word >> (8 * b));
  }
}

// ------------------------------------------------------------------ dense unpack
// llama/qlinear.py:120-162: dense[n, k] = cherry ? cherry_weight : fp16((q + 0.5) * s).
// A 32x32 (k, n) tile per block: codes are read with n contiguous, the dense matrix is
// written with k contiguous.
__global__ void unpack_dense_kernel(const uint8_t* __restrict__ q, const __half* __restrict__ scales,
                                    const __half* __restrict__ cw, const int16_t* __restrict__ idx,
                                    int bits, int K, int N, int C, int G, __half* __restrict__ dense) {
  __shared__ __half tile[32][33];
  const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
  for (int kk = ty; kk < 32; kk += 8) {
    const int k = k0 + kk, n = n0 + tx;
    __half v = __float2half(0.f);
    if (k < K && n < N) {
      // rank of k among the sorted cherry columns
      int low = 0, high = C;
      while (low < high) {
        const int mid = (low + high) >> 1;
        if ((int)idx[mid] < k) low = mid + 1; else high = mid;
      }
      if (low < C && (int)idx[low] == k) {
        v = cw[(size_t)low * N + n];
      } else {
        const int kc = k - low;
        const int u = (int)cq_ref_code(q, bits, kc, n, N);
        const __half a = __float2half_rn((float)(u - (1 << (bits - 1))) + 0.5f);
        v = __float2half_rn(__fmul_rn(__half2float(a), __half2float(scales[(size_t)(kc / G) * N + n])));
      }
    }
    tile[kk][tx] = v;
  }
  __syncthreads();
  for (int nn = ty; nn < 32; nn += 8) {
    const int n = n0 + nn, k = k0 + tx;
    if (k < K && n < N) dense[(size_t)n * K + k] = tile[tx][nn];
  }
}

// ------------------------------------------------------------------ Dequantize{3,4}Normal
__global__ void dequant_normal_kernel(const uint8_t* __restrict__ q, const float* __restrict__ sf,
                                      float* __restrict__ out, int bits, int Kc, int N, int G) {
  const long long total = (long long)Kc * N;
  const float off = (float)(1 << (bits - 1)) - 0.5f;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(id % N), kc = (int)(id / N);
    const float u = (float)cq_ref_code(q, bits, kc, n, N);
    out[id] = __fmul_rn(__fsub_rn(u, off), sf[(size_t)(kc / G) * N + n]);
  }
}

int nblocks(long long total, int threads) {
  long long b = (total + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > 148 * 32) b = 148 * 32;
  return (int)b;
}

int check_dims(int bits, int K, int N, int C, int* G) {
  if (bits != 3 && bits != 4) return CQ_ERR_BAD_BITS;
  if (*G == -1) *G = K;
  if (K <= 0 || N <= 0 || C < 0 || K % 8 || N % 8 || C % 8 || C >= K || K > 65534) return CQ_ERR_BAD_SHAPE;
  if (*G <= 0) return CQ_ERR_BAD_GROUP;
  return CQ_OK;
}

}  // namespace

extern "C" size_t cq_pack_tmp_bytes(int K) { (void)K; return 256; }

extern "C" int cq_pack(const void* weight, int weight_is_f32, const int32_t* cherry_unsorted, int bits,
                       int K, int N, int C, int G, uint8_t* qweight, void* scales, void* cherry_weight,
                       int16_t* cherry_indices, void* tmp, cq_stream_t stream) {
  (void)tmp;
  if (!weight || !qweight || !scales) return CQ_ERR_BAD_ARG;
  if (C > 0 && (!cherry_unsorted || !cherry_weight || !cherry_indices)) return CQ_ERR_BAD_ARG;
  const int rc = check_dims(bits, K, N, C, &G);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int T = 256;
  if (C > 0) {
    pack_sort_kernel<<<nblocks(C, T), T, 0, st>>>(cherry_unsorted, C, cherry_indices);
    pack_cherry_kernel<<<nblocks((long long)C * N, T), T, 0, st>>>(weight, weight_is_f32, cherry_indices, K, N, C,
                                                                  (__half*)cherry_weight);
  }
  const int ng = (K - C + G - 1) / G;
  pack_scales_kernel<<<nblocks((long long)ng * N * 32, T), T, 0, st>>>(weight, weight_is_f32, cherry_indices, bits,
                                                                      K, N, C, G, (__half*)scales);
  pack_codes_kernel<<<nblocks((long long)((K - C) / 8) * N, T), T, 0, st>>>(
      weight, weight_is_f32, cherry_indices, (const __half*)scales, bits, K, N, C, G, qweight);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}

extern "C" int cq_unpack_dense(const uint8_t* qweight, const void* scales, const void* cherry_weight,
                               const int16_t* cherry_indices, int bits, int K, int N, int C, int G,
                               void* dense, cq_stream_t stream) {
  if (!qweight || !scales || !dense) return CQ_ERR_BAD_ARG;
  if (C > 0 && (!cherry_weight || !cherry_indices)) return CQ_ERR_BAD_ARG;
  const int rc = check_dims(bits, K, N, C, &G);
  if (rc) return rc;
  dim3 grid((K + 31) / 32, (N + 31) / 32), block(32, 8);
  unpack_dense_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(qweight, (const __half*)scales,
                                                                (const __half*)cherry_weight, cherry_indices, bits,
                                                                K, N, C, G, (__half*)dense);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}

static int dequant_normal(int bits, const uint8_t* qweight, const float* sf, float* out, int qrows, int width,
                          int height, int cherry_size, int group_size, cq_stream_t stream) {
  if (!qweight || !sf || !out) return CQ_ERR_BAD_ARG;
  if (group_size == -1) group_size = height;
  if (width <= 0 || height <= 0 || cherry_size < 0 || cherry_size >= height || group_size <= 0)
    return CQ_ERR_BAD_SHAPE;
  const int Kc = height - cherry_size;
  if (Kc % 8 || qrows != Kc / 8 * bits) return CQ_ERR_BAD_SHAPE;
  dequant_normal_kernel<<<nblocks((long long)Kc * width, 256), 256, 0, (cudaStream_t)stream>>>(
      qweight, sf, out, bits, Kc, width, group_size);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}

extern "C" int cq_dequantize3_normal(const uint8_t* qweight, const float* sf, float* out, int qrows, int width,
                                     int height, int cherry_size, int group_size, cq_stream_t stream) {
  return dequant_normal(3, qweight, sf, out, qrows, width, height, cherry_size, group_size, stream);
}
extern "C" int cq_dequantize4_normal(const uint8_t* qweight, const float* sf, float* out, int qrows, int width,
                                     int height, int cherry_size, int group_size, cq_stream_t stream) {
  return dequant_normal(4, qweight, sf, out, qrows, width, height, cherry_size, group_size, stream);
}
