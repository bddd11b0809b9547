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

// Single-query attention over the KV cache (decode).  q and out are (sequences, H, D), the caches
// (sequences, max_seq, KV, D); positions 0..pos[sequence] take part (pos is read on the device, so
// the same launch serves every step of a captured graph).  A CTA handles one query head of one
// sequence (blockIdx.x, .y) and one of gridDim.z equal ranges of the positions: with one head per
// CTA alone a decode step would use H of the 148 SMs and crawl through a long context.  Each CTA
// computes its range's scores, their maximum m, the sum l of exp(score - m) and the unnormalised
// weighted sum of V; with one range that is the result, otherwise the CTA that finishes last (an
// atomic counter per head, which it resets) merges the ranges' (m, l, sum) from `part`.
// Scores and sums are fp32; a range's scores are held in shared memory.
constexpr int ATT_THREADS = 512, ATT_WARPS = ATT_THREADS / 32;
constexpr int ATT_MAX_SPLITS = 32;
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(const __half* __restrict__ q,
                                                                  const __half* __restrict__ k_cache,
                                                                  const __half* __restrict__ v_cache,
                                                                  const long long* __restrict__ pos,
                                                                  __half* __restrict__ out, float* __restrict__ part,
                                                                  unsigned int* __restrict__ counters, int H, int KV, int D,
                                                                  int max_seq, float scale) {
  // programmatic dependent launch: let the next kernel start its prologue, then wait for our inputs
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  extern __shared__ float sc[];              // [range] scores, then [ATT_THREADS] reduction scratch
  __shared__ int s_last;
  const int head = blockIdx.x, kvh = head / (H / KV), seq = blockIdx.y;
  const int split = blockIdx.z, nsplit = gridDim.z;
  q += (size_t)seq * H * D;
  out += (size_t)seq * H * D;
  k_cache += (size_t)seq * max_seq * KV * D;
  v_cache += (size_t)seq * max_seq * KV * D;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // positions beyond the cache are not attended to (the host refuses such steps; this keeps a stray
  // launch inside its shared-memory score array and the caches)
  const long long pl = pos[seq];
  const int n_all = pl < 0 ? 1 : (pl >= max_seq ? max_seq : (int)pl + 1);
  const int range = (max_seq + nsplit - 1) / nsplit;           // shared-memory scores per CTA
  const int chunk = (n_all + nsplit - 1) / nsplit;              // <= range
  const int pbeg = split * chunk;
  const int n_pos = max(0, min(n_all - pbeg, chunk));           // positions pbeg .. pbeg + n_pos - 1
  float* red = sc + range;
  const __half* qh = q + (size_t)head * D;
  const __half* kb = k_cache + ((size_t)pbeg * KV + kvh) * D;
  // scores: a warp per position, four positions in flight per warp, lanes over the head dimension
  float lmax = -INFINITY;
  for (int p0 = warp; p0 < n_pos; p0 += 4 * ATT_WARPS) {
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    const __half* kr[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int p = p0 + u * ATT_WARPS;
      kr[u] = kb + (size_t)(p < n_pos ? p : p0) * KV * D;
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
  __syncthreads();
  // weighted sum: thread (d, part) adds the positions p = part, part + parts, ... (D divides ATT_THREADS)
  const int parts = ATT_THREADS / D;
  const int d = tid % D, prt = tid / D;
  float acc0 = 0.f, acc1 = 0.f;
  {
    const __half* vb = v_cache + ((size_t)pbeg * KV + kvh) * D + d;
    const size_t vstride = (size_t)KV * D;
    int p = prt;
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
  float vsum = 0.f;
  if (tid < D)
    for (int i = 0; i < parts; ++i) vsum += red[tid + i * D];
  if (nsplit == 1) {
    if (tid < D) out[(size_t)head * D + tid] = __float2half(vsum / tot);
    return;
  }
  // ---- several ranges: publish (m, l, sum), the last CTA of this head merges
  const size_t hidx = (size_t)seq * H + head;
  float* mine = part + (hidx * nsplit + split) * (size_t)(D + 2);
  if (tid < D) mine[2 + tid] = vsum;
  if (tid == 0) { mine[0] = m; mine[1] = tot; }
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(&counters[hidx], 1u) == (unsigned int)(nsplit - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* all = part + hidx * nsplit * (size_t)(D + 2);
  float mm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, __ldcg(all + (size_t)s * (D + 2)));
  if (tid < D) {
    float l = 0.f, v = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float* ps = all + (size_t)s * (D + 2);
      const float ms = __ldcg(ps);
      const float w = ms == -INFINITY ? 0.f : __expf(ms - mm);       // an empty range carries no weight
      l += w * __ldcg(ps + 1);
      v += w * __ldcg(ps + 2 + tid);
    }
    out[(size_t)head * D + tid] = __float2half(v / l);
  }
  if (tid == 0) counters[hidx] = 0u;                                  // ready for the next launch
}

// The same for grouped-query models and long caches: one CTA per KV head (blockIdx.x), sequence and range
// of positions handles all G = H / KV query heads that share the KV head, so every K and V row is read
// once (with one CTA per query head it is read G times through L2).  A group of D / 8 lanes takes one
// position with 16-byte loads (8 values a lane), GT >= G query heads at a time in registers.  Partial
// results of the ranges as in the kernel above; the arrival counter is per (sequence, KV head).
constexpr int GQA_THREADS = 256, GQA_WARPS = GQA_THREADS / 32;
template <int GT>
__global__ void __launch_bounds__(GQA_THREADS) attn_decode_gqa_kernel(const __half* __restrict__ q,
                                                                      const __half* __restrict__ k_cache,
                                                                      const __half* __restrict__ v_cache,
                                                                      const long long* __restrict__ pos,
                                                                      __half* __restrict__ out, float* __restrict__ part,
                                                                      unsigned int* __restrict__ counters, int H, int KV,
                                                                      int D, int max_seq, float scale) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  extern __shared__ float sm[];              // [GT][range] scores, later [warps][GT][D] partial sums of V
  __shared__ float s_m[GT], s_l[GT];
  __shared__ int s_last;
  const int kvh = blockIdx.x, seq = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
  const int G = H / KV, head0 = kvh * G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int lpp = D >> 3;                    // lanes per position: 8, 16 or 32
  const int ppw = 32 / lpp;                  // positions a warp takes per turn
  const int sub = lane / lpp, l = lane - sub * lpp;
  const long long pl = pos[seq];
  const int n_all = pl < 0 ? 1 : (pl >= max_seq ? max_seq : (int)pl + 1);
  const int range = (max_seq + nsplit - 1) / nsplit;
  const int chunk = (n_all + nsplit - 1) / nsplit;
  const int pbeg = split * chunk;
  const int n_pos = max(0, min(n_all - pbeg, chunk));
  const size_t row = (size_t)KV * D;         // elements between consecutive positions of a cache
  const __half* kb = k_cache + ((size_t)seq * max_seq + pbeg) * row + (size_t)kvh * D + l * 8;
  const __half* vb = v_cache + ((size_t)seq * max_seq + pbeg) * row + (size_t)kvh * D + l * 8;

  // ---- scores
  {
    uint4 qr[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g)
      qr[g] = g < G ? *reinterpret_cast<const uint4*>(q + ((size_t)seq * H + head0 + g) * D + l * 8) : make_uint4(0, 0, 0, 0);
    const int stride = GQA_WARPS * ppw;
    constexpr int UF = 4;                                 // positions per lane group in flight (loads first, then math)
    for (int base = warp * ppw; base < n_pos; base += UF * stride) {
      uint4 kk[UF];
#pragma unroll
      for (int j = 0; j < UF; ++j) {
        const int pj = base + sub + j * stride;
        kk[j] = pj < n_pos ? __ldg(reinterpret_cast<const uint4*>(kb + (size_t)pj * row)) : make_uint4(0, 0, 0, 0);
      }
      float2 kf[UF][4];                                   // converted once, used by every query head
#pragma unroll
      for (int j = 0; j < UF; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) kf[j][i] = __half22float2(reinterpret_cast<const __half2*>(&kk[j])[i]);
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        if (g < G) {
          const __half2* qh = reinterpret_cast<const __half2*>(&qr[g]);
          float2 qf[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) qf[i] = __half22float2(qh[i]);
          float d[UF];
#pragma unroll
          for (int j = 0; j < UF; ++j) {
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) a += qf[i].x * kf[j][i].x + qf[i].y * kf[j][i].y;
            d[j] = a;
          }
          for (int o = lpp >> 1; o > 0; o >>= 1) {
#pragma unroll
            for (int j = 0; j < UF; ++j) d[j] += __shfl_xor_sync(0xffffffffu, d[j], o);
          }
          if (l == 0) {
#pragma unroll
            for (int j = 0; j < UF; ++j) {
              const int pj = base + sub + j * stride;
              if (pj < n_pos) sm[g * range + pj] = d[j] * scale;
            }
          }
        }
      }
    }
  }
  __syncthreads();
  // ---- softmax pieces: warp g takes query head g (GT <= number of warps)
  if (warp < G) {
    float* sg = sm + warp * range;
    float m = -INFINITY;
    for (int p = lane; p < n_pos; p += 32) m = fmaxf(m, sg[p]);
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
    for (int p = lane; p < n_pos; p += 32) {
      const float e = __expf(sg[p] - m);
      sg[p] = e;
      sum += e;
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) { s_m[warp] = m; s_l[warp] = sum; }
  }
  __syncthreads();
  // ---- weighted sums of V: a lane keeps 8 head-dimension values of every query head
  float acc[GT][8];
#pragma unroll
  for (int g = 0; g < GT; ++g)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  {
    const int stride = GQA_WARPS * ppw;
    constexpr int UF = 4;
    for (int base = warp * ppw; base < n_pos; base += UF * stride) {
      uint4 vv[UF];
#pragma unroll
      for (int j = 0; j < UF; ++j) {
        const int pj = base + sub + j * stride;
        vv[j] = pj < n_pos ? __ldg(reinterpret_cast<const uint4*>(vb + (size_t)pj * row)) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < UF; ++j) {
        const int pj = base + sub + j * stride;
        const bool ok = pj < n_pos;
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 a = __half22float2(reinterpret_cast<const __half2*>(&vv[j])[i]);
          f[2 * i] = a.x; f[2 * i + 1] = a.y;
        }
#pragma unroll
        for (int g = 0; g < GT; ++g) {
          if (g < G) {
            const float w = ok ? sm[g * range + pj] : 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[g][i] += w * f[i];
          }
        }
      }
    }
  }
  // the position groups of a warp hold the same head-dimension values: add them (lanes l of every group)
#pragma unroll
  for (int g = 0; g < GT; ++g)
#pragma unroll
    for (int i = 0; i < 8; ++i)
      for (int o = lpp; o < 32; o <<= 1) acc[g][i] += __shfl_xor_sync(0xffffffffu, acc[g][i], o);
  __syncthreads();                                     // every warp is done with the scores: the memory is re-used
  float* red = sm;                                     // [warps][GT][D]
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < GT; ++g)
      if (g < G)
#pragma unroll
        for (int i = 0; i < 8; ++i) red[((size_t)warp * GT + g) * D + l * 8 + i] = acc[g][i];
  }
  __syncthreads();
  const size_t hbase = (size_t)seq * H + head0;
  for (int e = tid; e < G * D; e += GQA_THREADS) {
    const int g = e / D, d = e - g * D;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < GQA_WARPS; ++w) v += red[((size_t)w * GT + g) * D + d];
    if (nsplit == 1) {
      out[(hbase + g) * D + d] = __float2half(v / s_l[g]);
    } else {
      float* mine = part + ((hbase + g) * nsplit + split) * (size_t)(D + 2);
      mine[2 + d] = v;
      if (d == 0) { mine[0] = s_m[g]; mine[1] = s_l[g]; }
    }
  }
  if (nsplit == 1) return;
  __threadfence();
  __syncthreads();
  const size_t cidx = (size_t)seq * KV + kvh;
  if (tid == 0) s_last = atomicAdd(&counters[cidx], 1u) == (unsigned int)(nsplit - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int e = tid; e < G * D; e += GQA_THREADS) {
    const int g = e / D, d = e - g * D;
    const float* all = part + (hbase + g) * nsplit * (size_t)(D + 2);
    float mm = -INFINITY;
    for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, __ldcg(all + (size_t)s * (D + 2)));
    float lsum = 0.f, v = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float* ps = all + (size_t)s * (D + 2);
      const float ms = __ldcg(ps);
      const float w = ms == -INFINITY ? 0.f : __expf(ms - mm);       // an empty range carries no weight
      lsum += w * __ldcg(ps + 1);
      v += w * __ldcg(ps + 2 + d);
    }
    out[(hbase + g) * D + d] = __float2half(v / lsum);
  }
  if (tid == 0) counters[cidx] = 0u;                                  // ready for the next launch
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

namespace {
// ranges of positions per head: enough CTAs for about two per SM, at least 256 cache positions per range
int attn_splits(int sequences, int n_heads, int max_seq) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int s = (2 * sms + sequences * n_heads - 1) / (sequences * n_heads);
  const int by_len = (max_seq + 255) / 256;
  if (s > by_len) s = by_len;
  if (s > ATT_MAX_SPLITS) s = ATT_MAX_SPLITS;
  return s < 1 ? 1 : s;
}
}  // namespace

extern "C" size_t cq_attn_decode_workspace_bytes(int sequences, int n_heads, int head_dim, int max_seq) {
  if (sequences < 1 || n_heads < 1 || head_dim < 2 || max_seq < 1) return 0;
  const size_t heads = (size_t)sequences * n_heads;
  // [heads] counters (zero before the first use; every launch leaves them zero), then the ranges' partial results
  // (the grouped-query kernel divides by KV heads and may use more ranges than the per-head one: room for the maximum)
  return heads * sizeof(unsigned int) + 256 + heads * ATT_MAX_SPLITS * (size_t)(head_dim + 2) * sizeof(float);
}

extern "C" int cq_attn_decode(const void* q, const void* k_cache, const void* v_cache, const long long* position,
                              void* out, int sequences, int n_heads, int n_kv_heads, int head_dim, int max_seq,
                              float scale, void* workspace, cq_stream_t stream) {
  if (!q || !k_cache || !v_cache || !position || !out || !workspace || sequences < 1 || sequences > 65535) return CQ_ERR_BAD_ARG;
  if ((uintptr_t)workspace & 15) return CQ_ERR_BAD_ARG;
  if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads || head_dim < 2 || head_dim > 256 || (head_dim & 1) ||
      256 % head_dim || max_seq < 1 || max_seq > 65536)
    return CQ_ERR_BAD_SHAPE;
  const size_t heads = (size_t)sequences * n_heads;
  unsigned int* counters = (unsigned int*)workspace;
  float* part = (float*)((uint8_t*)workspace + (heads * sizeof(unsigned int) + 255) / 256 * 256);
  const int G = n_heads / n_kv_heads;
  // One CTA per KV head reads every cache row once for the query heads that share it; with several query heads
  // per KV head its per-position arithmetic is G times larger, which only pays on long caches (measured, 70B
  // shapes: 103 us against 174 at 4000 positions, but 21 against 15 at 200): short grouped-query caches keep
  // the per-head kernel, whose re-reads hit L2.
  if ((head_dim == 64 || head_dim == 128 || head_dim == 256) && G <= 8 && (G == 1 || max_seq > 1024)) {
    const int splits = attn_splits(sequences, n_kv_heads, max_seq);
    const int range = (max_seq + splits - 1) / splits;
    const int gt = G <= 1 ? 1 : (G <= 2 ? 2 : (G <= 4 ? 4 : 8));
    const int words = gt * range > GQA_WARPS * gt * head_dim ? gt * range : GQA_WARPS * gt * head_dim;
    const int smem = words * (int)sizeof(float);
    if (smem > 200 * 1024) return CQ_ERR_TOO_LARGE;
    void (*fn)(const __half*, const __half*, const __half*, const long long*, __half*, float*, unsigned int*, int, int, int, int, float) =
        gt == 1 ? attn_decode_gqa_kernel<1> : (gt == 2 ? attn_decode_gqa_kernel<2> : (gt == 4 ? attn_decode_gqa_kernel<4> : attn_decode_gqa_kernel<8>));
    if (smem > 48 * 1024) CQ_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    CQ_CUDA_TRY(launch_pdl(fn, dim3(n_kv_heads, sequences, splits), dim3(GQA_THREADS), (size_t)smem, (cudaStream_t)stream,
                           (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, position, (__half*)out, part,
                           counters, n_heads, n_kv_heads, head_dim, max_seq, scale));
    return CQ_OK;
  }
  const int splits = attn_splits(sequences, n_heads, max_seq);
  const int range = (max_seq + splits - 1) / splits;
  const int smem = (range + ATT_THREADS) * (int)sizeof(float);
  if (smem > 200 * 1024) return CQ_ERR_TOO_LARGE;
  if (smem > 48 * 1024)
    CQ_CUDA_TRY(cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  CQ_CUDA_TRY(launch_pdl(attn_decode_kernel, dim3(n_heads, sequences, splits), dim3(ATT_THREADS), (size_t)smem,
                         (cudaStream_t)stream, (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, position,
                         (__half*)out, part, counters, n_heads, n_kv_heads, head_dim, max_seq, scale));
  return CQ_OK;
}
