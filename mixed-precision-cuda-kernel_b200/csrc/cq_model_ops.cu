// Small fused element-wise kernels of the decode harness around the quantized linear: RMSNorm with
// the residual add, rotary embedding + KV-cache write, SwiGLU gate.  In the reference these are
// separate PyTorch ops of its vendored LLaMA (llama/modeling_llama_quant.py: LlamaRMSNorm,
// apply_rotary_pos_emb, LlamaMLP.forward of the reference project); at batch 1 each of them is a
// launch-latency-bound kernel, so the harness fuses them to keep the step dominated by the
// projections.  fp16 in / out, fp32 arithmetic.
#include "cq_common.cuh"

namespace {

// One CTA per row: h = x (+ residual); y = h * rsqrt(mean(h^2) + eps) * w; optionally h is stored.
// A thread keeps its (up to 16) values in registers between the two passes; 16-byte accesses.
// hidden is a multiple of 8 and at most 16 * 1024.
__global__ void __launch_bounds__(1024) rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ residual,
                                                       const __half* __restrict__ w, __half* __restrict__ y,
                                                       __half* __restrict__ h_out, int hidden, float eps) {
  // programmatic dependent launch: let the next kernel start its prologue, then wait for our inputs
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const int nvec = hidden >> 3;                       // 16-byte vectors per row
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * hidden);
  const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + row * hidden) : nullptr;
  uint4 hv[2];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    hv[c] = make_uint4(0, 0, 0, 0);
    if (i < nvec) {
      uint4 v = xr[i];
      if (rr) {
        const uint4 r = rr[i];
        __half2* a = reinterpret_cast<__half2*>(&v);
        const __half2* b = reinterpret_cast<const __half2*>(&r);
#pragma unroll
        for (int e = 0; e < 4; ++e) a[e] = __hadd2(a[e], b[e]);            // the sum is an fp16 tensor
      }
      hv[c] = v;
      const __half2* a = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(a[e]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)hidden + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nvec) {
      if (h_out) reinterpret_cast<uint4*>(h_out + row * hidden)[i] = hv[c];
      const uint4 wv = wr[i];
      uint4 o;
      const __half2* a = reinterpret_cast<const __half2*>(&hv[c]);
      const __half2* ww = reinterpret_cast<const __half2*>(&wv);
      __half2* oo = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(a[e]);
        oo[e] = __hmul2(__floats2half2_rn(f.x * inv, f.y * inv), ww[e]);
      }
      reinterpret_cast<uint4*>(y + row * hidden)[i] = o;
    }
  }
}

// Rotary embedding ("rotate half" convention) of q (T, H, D) and k (T, KV, D) in place at positions
// pos[t], and the write of k, v rows into the caches (sequences, max_seq, KV, D): token t belongs to
// sequence t / tokens_per_seq.
__global__ void rope_cache_kernel(__half* __restrict__ q, __half* __restrict__ k, const __half* __restrict__ v,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  const long long* __restrict__ pos, __half* __restrict__ k_cache,
                                  __half* __restrict__ v_cache, int T, int H, int KV, int D, int max_seq,
                                  int tokens_per_seq) {
  // programmatic dependent launch: let the next kernel start its prologue, then wait for our inputs
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int half = D / 2;
  const long long total = (long long)T * (H + 2 * KV) * half;
  for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total;
       id += (long long)gridDim.x * blockDim.x) {
    const int i = (int)(id % half);
    const int hh = (int)((id / half) % (H + 2 * KV));
    const int t = (int)(id / ((long long)half * (H + 2 * KV)));
    const long long p = pos[t];
    if (p < 0 || p >= max_seq) continue;      // a position outside the tables and caches: nothing is read or written
    const size_t crow = (size_t)(t / tokens_per_seq) * max_seq + (size_t)p;     // row of the caches
    if (hh < H + KV) {
      __half* base = hh < H ? q + ((size_t)t * H + hh) * D : k + ((size_t)t * KV + (hh - H)) * D;
      const float c = cos_t[p * half + i], s = sin_t[p * half + i];
      const float x1 = __half2float(base[i]), x2 = __half2float(base[i + half]);
      const __half o1 = __float2half(x1 * c - x2 * s), o2 = __float2half(x2 * c + x1 * s);
      base[i] = o1;
      base[i + half] = o2;
      if (hh >= H) {
        __half* kc = k_cache + (crow * KV + (hh - H)) * D;
        kc[i] = o1;
        kc[i + half] = o2;
      }
    } else {
      const int kvh = hh - H - KV;
      const __half* src = v + ((size_t)t * KV + kvh) * D;
      __half* vc = v_cache + (crow * KV + kvh) * D;
      vc[i] = src[i];
      vc[i + half] = src[i + half];
    }
  }
}

__global__ void silu_mul_kernel(const __half* __restrict__ gate, const __half* __restrict__ up,
                                __half* __restrict__ out, long long n) {
  // programmatic dependent launch: let the next kernel start its prologue, then wait for our inputs
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float g = __half2float(gate[i]);
    const __half act = __float2half(g / (1.f + __expf(-g)));          // silu result is an fp16 tensor
    out[i] = __hmul(act, up[i]);
  }
}

// Single-query attention over the KV cache (decode): one CTA per query head and sequence (blockIdx.y);
// q and out are (sequences, H, D), the caches (sequences, max_seq, KV, D).  Positions 0..pos[sequence]
// take part (pos is read on the device, so the same launch serves every step of a captured graph).
// Scores and the weighted sum are fp32; softmax over at most `max_seq` positions held in shared memory.
constexpr int ATT_THREADS = 1024, ATT_WARPS = ATT_THREADS / 32;
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(const __half* __restrict__ q,
                                                                  const __half* __restrict__ k_cache,
                                                                  const __half* __restrict__ v_cache,
                                                                  const long long* __restrict__ pos,
                                                                  __half* __restrict__ out, int H, int KV, int D,
                                                                  int max_seq, float scale) {
  // programmatic dependent launch: let the next kernel start its prologue, then wait for our inputs
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  extern __shared__ float sc[];              // [n_pos] scores, then [ATT_THREADS] reduction scratch
  const int head = blockIdx.x, kvh = head / (H / KV), seq = blockIdx.y;
  q += (size_t)seq * H * D;
  out += (size_t)seq * H * D;
  k_cache += (size_t)seq * max_seq * KV * D;
  v_cache += (size_t)seq * max_seq * KV * D;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // positions beyond the cache are not attended to (the host refuses such steps; this keeps a stray
  // launch inside its shared-memory score array and the caches)
  const long long p0 = pos[seq];
  const int n_pos = p0 < 0 ? 1 : (p0 >= max_seq ? max_seq : (int)p0 + 1);
  float* red = sc + n_pos;
  const __half* qh = q + (size_t)head * D;
  // scores: a warp per position, four positions in flight per warp, lanes over the head dimension
  float lmax = -INFINITY;
  for (int p0 = warp; p0 < n_pos; p0 += 4 * ATT_WARPS) {
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    const __half* kr[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int p = p0 + u * ATT_WARPS;
      kr[u] = k_cache + ((size_t)(p < n_pos ? p : p0) * KV + kvh) * D;
    }
    for (int d = 2 * lane; d < D; d += 64) {
      const float2 qv = __half22float2(*reinterpret_cast<const __half2*>(qh + d));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 kv2 = __half22float2(*reinterpret_cast<const __half2*>(kr[u] + d));
        a[u] += qv.x * kv2.x + qv.y * kv2.y;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      for (int o = 16; o > 0; o >>= 1) a[u] += __shfl_xor_sync(0xffffffffu, a[u], o);
      a[u] *= scale;
      const int p = p0 + u * ATT_WARPS;
      if (p < n_pos) {
        if (lane == 0) sc[p] = a[u];
        lmax = fmaxf(lmax, a[u]);
      }
    }
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
  {
    const __half* vb = v_cache + (size_t)kvh * D + d;
    const size_t vstride = (size_t)KV * D;
    int p = part;
    for (; p + 7 * parts < n_pos; p += 8 * parts) {       // eight loads in flight
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __half2float(vb[(size_t)(p + u * parts) * vstride]);
#pragma unroll
      for (int u = 0; u < 8; u += 2) {
        acc0 += sc[p + u * parts] * v[u];
        acc1 += sc[p + (u + 1) * parts] * v[u + 1];
      }
    }
    for (; p < n_pos; p += parts) acc0 += sc[p] * __half2float(vb[(size_t)p * vstride]);
  }
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

// All kernels here are launched with the programmatic-serialization attribute (they wait for their
// inputs with griddepcontrol.wait), so that in a chain of small kernels the launch latencies overlap.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace

extern "C" int cq_rmsnorm(const void* x, const void* residual, const void* weight, void* y, void* h_out, int rows,
                          int hidden, float eps, cq_stream_t stream) {
  if (!x || !weight || !y || rows < 1 || hidden < 8) return CQ_ERR_BAD_ARG;
  if ((hidden & 7) || hidden > 16 * 1024) return CQ_ERR_BAD_SHAPE;
  if (((uintptr_t)x | (uintptr_t)weight | (uintptr_t)y | (uintptr_t)residual | (uintptr_t)h_out) & 15) return CQ_ERR_BAD_ARG;
  int threads = ((hidden >> 3) + 1) / 2;                 // two 16-byte vectors per thread
  threads = (threads + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  if (threads < 32) threads = 32;
  CQ_CUDA_TRY(launch_pdl(rmsnorm_kernel, dim3(rows), dim3(threads), 0, (cudaStream_t)stream, (const __half*)x,
                         (const __half*)residual, (const __half*)weight, (__half*)y, (__half*)h_out, hidden, eps));
  return CQ_OK;
}

extern "C" int cq_rope_cache(void* q, void* k, const void* v, const float* cos_table, const float* sin_table,
                             const long long* positions, void* k_cache, void* v_cache, int T, int n_heads,
                             int n_kv_heads, int head_dim, int max_seq, int tokens_per_seq, cq_stream_t stream) {
  if (tokens_per_seq < 1 || T % tokens_per_seq) return CQ_ERR_BAD_ARG;
  if (!q || !k || !v || !cos_table || !sin_table || !positions || !k_cache || !v_cache) return CQ_ERR_BAD_ARG;
  if (T < 1 || n_heads < 1 || n_kv_heads < 1 || head_dim < 2 || (head_dim & 1) || max_seq < 1) return CQ_ERR_BAD_ARG;
  const long long total = (long long)T * (n_heads + 2 * n_kv_heads) * (head_dim / 2);
  CQ_CUDA_TRY(launch_pdl(rope_cache_kernel, dim3(blocks_for(total, 256, 148 * 8)), dim3(256), 0, (cudaStream_t)stream,
                         (__half*)q, (__half*)k, (const __half*)v, cos_table, sin_table, positions, (__half*)k_cache,
                         (__half*)v_cache, T, n_heads, n_kv_heads, head_dim, max_seq, tokens_per_seq));
  return CQ_OK;
}

extern "C" int cq_silu_mul(const void* gate, const void* up, void* out, long long n, cq_stream_t stream) {
  if (!gate || !up || !out || n < 1) return CQ_ERR_BAD_ARG;
  CQ_CUDA_TRY(launch_pdl(silu_mul_kernel, dim3(blocks_for(n, 256, 148 * 8)), dim3(256), 0, (cudaStream_t)stream,
                         (const __half*)gate, (const __half*)up, (__half*)out, n));
  return CQ_OK;
}

extern "C" int cq_attn_decode(const void* q, const void* k_cache, const void* v_cache, const long long* position,
                              void* out, int sequences, int n_heads, int n_kv_heads, int head_dim, int max_seq,
                              float scale, cq_stream_t stream) {
  if (!q || !k_cache || !v_cache || !position || !out || sequences < 1 || sequences > 65535) return CQ_ERR_BAD_ARG;
  if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads || head_dim < 2 || head_dim > 256 || (head_dim & 1) ||
      256 % head_dim || max_seq < 1 || max_seq > 8192)
    return CQ_ERR_BAD_SHAPE;
  const int smem = (max_seq + ATT_THREADS) * (int)sizeof(float);
  CQ_CUDA_TRY(launch_pdl(attn_decode_kernel, dim3(n_heads, sequences), dim3(ATT_THREADS), (size_t)smem, (cudaStream_t)stream,
                         (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, position, (__half*)out, n_heads,
                         n_kv_heads, head_dim, max_seq, scale));
  return CQ_OK;
}
