// Small fused element-wise kernels of the decode harness around the quantized linear: RMSNorm with
// the residual add, rotary embedding + KV-cache write, SwiGLU gate.  In the reference these are
// separate PyTorch ops of its vendored LLaMA (llama/modeling_llama_quant.py: LlamaRMSNorm,
// apply_rotary_pos_emb, LlamaMLP.forward of the reference project); at batch 1 each of them is a
// launch-latency-bound kernel, so the harness fuses them to keep the step dominated by the
// projections.  fp16 in / out, fp32 arithmetic.
#include "cq_common.cuh"

namespace {

// One CTA per row: h = x (+ residual); y = h * rsqrt(mean(h^2) + eps) * w; optionally h is stored.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ residual,
                                                      const __half* __restrict__ w, __half* __restrict__ y,
                                                      __half* __restrict__ h_out, int hidden, float eps) {
  __shared__ float red[8];
  const size_t row = blockIdx.x;
  const __half* xr = x + row * hidden;
  const __half* rr = residual ? residual + row * hidden : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = __half2float(xr[i]);
    if (rr) v = __half2float(__float2half(v + __half2float(rr[i])));   // the sum is an fp16 tensor
    ss += v * v;
  }
  for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = __half2float(xr[i]);
    if (rr) v = __half2float(__float2half(v + __half2float(rr[i])));
    if (h_out) h_out[row * hidden + i] = __float2half(v);
    y[row * hidden + i] = __hmul(__float2half(v * inv), w[i]);
  }
}

// Rotary embedding ("rotate half" convention) of q (T, H, D) and k (T, KV, D) in place at positions
// pos[t], and the write of k, v rows into the caches (max_seq, KV, D).
__global__ void rope_cache_kernel(__half* __restrict__ q, __half* __restrict__ k, const __half* __restrict__ v,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  const long long* __restrict__ pos, __half* __restrict__ k_cache,
                                  __half* __restrict__ v_cache, int T, int H, int KV, int D) {
  const int half = D / 2;
  const long long total = (long long)T * (H + 2 * KV) * half;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int i = (int)(id % half);
    const int hh = (int)((id / half) % (H + 2 * KV));
    const int t = (int)(id / ((long long)half * (H + 2 * KV)));
    const long long p = pos[t];
    if (hh < H + KV) {
      __half* base = hh < H ? q + ((size_t)t * H + hh) * D : k + ((size_t)t * KV + (hh - H)) * D;
      const float c = cos_t[p * half + i], s = sin_t[p * half + i];
      const float x1 = __half2float(base[i]), x2 = __half2float(base[i + half]);
      const __half o1 = __float2half(x1 * c - x2 * s), o2 = __float2half(x2 * c + x1 * s);
      base[i] = o1;
      base[i + half] = o2;
      if (hh >= H) {
        __half* kc = k_cache + ((size_t)p * KV + (hh - H)) * D;
        kc[i] = o1;
        kc[i + half] = o2;
      }
    } else {
      const int kvh = hh - H - KV;
      const __half* src = v + ((size_t)t * KV + kvh) * D;
      __half* vc = v_cache + ((size_t)p * KV + kvh) * D;
      vc[i] = src[i];
      vc[i + half] = src[i + half];
    }
  }
}

__global__ void silu_mul_kernel(const __half* __restrict__ gate, const __half* __restrict__ up,
                                __half* __restrict__ out, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float g = __half2float(gate[i]);
    const __half act = __float2half(g / (1.f + __expf(-g)));          // silu result is an fp16 tensor
    out[i] = __hmul(act, up[i]);
  }
}

// Single-query attention over the KV cache (decode): one CTA per query head.  Positions 0..pos[0]
// take part (pos is read on the device, so the same launch serves every step of a captured graph).
// Scores and the weighted sum are fp32; softmax over at most `max_seq` positions held in shared memory.
constexpr int ATT_THREADS = 1024, ATT_WARPS = ATT_THREADS / 32;
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(const __half* __restrict__ q,
                                                                  const __half* __restrict__ k_cache,
                                                                  const __half* __restrict__ v_cache,
                                                                  const long long* __restrict__ pos,
                                                                  __half* __restrict__ out, int H, int KV, int D,
                                                                  float scale) {
  extern __shared__ float sc[];              // [n_pos] scores, then [ATT_THREADS] reduction scratch
  const int head = blockIdx.x, kvh = head / (H / KV);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_pos = (int)pos[0] + 1;
  float* red = sc + n_pos;
  const __half* qh = q + (size_t)head * D;
  // scores: a warp per position (two positions in flight per warp), lanes over the head dimension
  float lmax = -INFINITY;
  for (int p0 = warp; p0 < n_pos; p0 += 2 * ATT_WARPS) {
    const int p1 = p0 + ATT_WARPS;
    const bool two = p1 < n_pos;
    const __half* k0 = k_cache + ((size_t)p0 * KV + kvh) * D;
    const __half* k1 = k_cache + ((size_t)(two ? p1 : p0) * KV + kvh) * D;
    float a0 = 0.f, a1 = 0.f;
    for (int d = 2 * lane; d < D; d += 64) {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(qh + d));
      const float2 b0 = __half22float2(*reinterpret_cast<const __half2*>(k0 + d));
      const float2 b1 = __half22float2(*reinterpret_cast<const __half2*>(k1 + d));
      a0 += a.x * b0.x + a.y * b0.y;
      a1 += a.x * b1.x + a.y * b1.y;
    }
    for (int o = 16; o > 0; o >>= 1) {
      a0 += __shfl_xor_sync(0xffffffffu, a0, o);
      a1 += __shfl_xor_sync(0xffffffffu, a1, o);
    }
    a0 *= scale;
    a1 *= scale;
    if (lane == 0) {
      sc[p0] = a0;
      if (two) sc[p1] = a1;
    }
    lmax = fmaxf(lmax, two ? fmaxf(a0, a1) : a0);
  }
  if (lane == 0) red[warp] = lmax;
  __syncthreads();
  float m = red[0];
  for (int i = 1; i < ATT_WARPS; ++i) m = fmaxf(m, red[i]);
  __syncthreads();
  float lsum = 0.f;
  for (int p = tid; p < n_pos; p += ATT_THREADS) {
    const float e = __expf(sc[p] - m);
    sc[p] = e;
    lsum += e;
  }
  for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
  if (lane == 0) red[warp] = lsum;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < ATT_WARPS; ++i) tot += red[i];
  const float inv = 1.f / tot;
  __syncthreads();
  // weighted sum: thread (d, part) adds the positions p = part, part + parts, ... (D divides ATT_THREADS)
  const int parts = ATT_THREADS / D;
  const int d = tid % D, part = tid / D;
  float acc0 = 0.f, acc1 = 0.f;
  int p = part;
  for (; p + parts < n_pos; p += 2 * parts) {
    acc0 += sc[p] * __half2float(v_cache[((size_t)p * KV + kvh) * D + d]);
    acc1 += sc[p + parts] * __half2float(v_cache[((size_t)(p + parts) * KV + kvh) * D + d]);
  }
  if (p < n_pos) acc0 += sc[p] * __half2float(v_cache[((size_t)p * KV + kvh) * D + d]);
  red[tid] = acc0 + acc1;
  __syncthreads();
  if (tid < D) {
    float v = 0.f;
    for (int i = 0; i < parts; ++i) v += red[tid + i * D];
    out[(size_t)head * D + tid] = __float2half(v * inv);
  }
}

int blocks_for(long long total, int threads, int cap) {
  long long b = (total + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > cap) b = cap;
  return (int)b;
}

}  // namespace

extern "C" int cq_rmsnorm(const void* x, const void* residual, const void* weight, void* y, void* h_out, int rows,
                          int hidden, float eps, cq_stream_t stream) {
  if (!x || !weight || !y || rows < 1 || hidden < 1) return CQ_ERR_BAD_ARG;
  rmsnorm_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>((const __half*)x, (const __half*)residual,
                                                           (const __half*)weight, (__half*)y, (__half*)h_out, hidden, eps);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}

extern "C" int cq_rope_cache(void* q, void* k, const void* v, const float* cos_table, const float* sin_table,
                             const long long* positions, void* k_cache, void* v_cache, int T, int n_heads,
                             int n_kv_heads, int head_dim, cq_stream_t stream) {
  if (!q || !k || !v || !cos_table || !sin_table || !positions || !k_cache || !v_cache) return CQ_ERR_BAD_ARG;
  if (T < 1 || n_heads < 1 || n_kv_heads < 1 || head_dim < 2 || (head_dim & 1)) return CQ_ERR_BAD_ARG;
  const long long total = (long long)T * (n_heads + 2 * n_kv_heads) * (head_dim / 2);
  rope_cache_kernel<<<blocks_for(total, 256, 148 * 8), 256, 0, (cudaStream_t)stream>>>(
      (__half*)q, (__half*)k, (const __half*)v, cos_table, sin_table, positions, (__half*)k_cache, (__half*)v_cache, T,
      n_heads, n_kv_heads, head_dim);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}

extern "C" int cq_silu_mul(const void* gate, const void* up, void* out, long long n, cq_stream_t stream) {
  if (!gate || !up || !out || n < 1) return CQ_ERR_BAD_ARG;
  silu_mul_kernel<<<blocks_for(n, 256, 148 * 8), 256, 0, (cudaStream_t)stream>>>((const __half*)gate, (const __half*)up,
                                                                                 (__half*)out, n);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}

extern "C" int cq_attn_decode(const void* q, const void* k_cache, const void* v_cache, const long long* position,
                              void* out, int n_heads, int n_kv_heads, int head_dim, int max_seq, float scale,
                              cq_stream_t stream) {
  if (!q || !k_cache || !v_cache || !position || !out) return CQ_ERR_BAD_ARG;
  if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads || head_dim < 2 || head_dim > 256 || (head_dim & 1) ||
      256 % head_dim || max_seq < 1 || max_seq > 8192)
    return CQ_ERR_BAD_SHAPE;
  const int smem = (max_seq + ATT_THREADS) * (int)sizeof(float);
  attn_decode_kernel<<<n_heads, ATT_THREADS, smem, (cudaStream_t)stream>>>((const __half*)q, (const __half*)k_cache,
                                                                   (const __half*)v_cache, position, (__half*)out,
                                                                   n_heads, n_kv_heads, head_dim, scale);
  CQ_CUDA_TRY(cudaGetLastError());
  return CQ_OK;
}
