// extern "C" entry points that keep the reference's operator signatures
// (csrc/quant_cuda.cpp:41-69 of the reference project) on top of the prepared
// layer interfaces: the first call with a given set of reference buffers re-packs
// them on the GPU into the layout of the kernel that serves the call's batch size
// and caches the result.  One activation row: row-tile layout (cq_rlayer) when the
// layer fits that kernel; 2..7 rows (and the layers it does not fit): stream layout
// (cq_layer); 8 rows or more (large decode batches, prefill): tile layout and the
// tensor-core GEMM.  A layer only pays for the layouts it is actually called with.
// cq_cache_evict drops the copies of one buffer set (the torch shim calls it when
// the tensors behind a cached address have been freed).
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "cq_common.cuh"

int cq_launch_matvec_f32(int bits, const float* x, const uint8_t* q, const float* cw, const int32_t* idx,
                         const float* sf, float* mul, int M, int K, int N, int C, int G, cudaStream_t st);

namespace {

thread_local int g_last_cuda_error = 0;

struct CacheKey {
  int dev;
  const void *q, *s, *cw, *idx;
  int bits, K, N, C, G;
  uint64_t tag;
  bool operator<(const CacheKey& o) const {
    return std::tie(dev, q, s, cw, idx, bits, K, N, C, G, tag) <
           std::tie(o.dev, o.q, o.s, o.cw, o.idx, o.bits, o.K, o.N, o.C, o.G, o.tag);
  }
};

struct DeviceState {
  void* scratch = nullptr;
  uint32_t* status = nullptr;
  void* gemm_ws = nullptr;        // staged activations of the prefill GEMM (grow-only)
  size_t gemm_ws_bytes = 0;
};

// From here on the tensor-core GEMM is used: measured on 4096 -> 11008 4-bit, 16 rows take 51 us on the
// stream matvec (whose per-row activation staging grows with the batch) and 34 us on the GEMM with
// split-K; at 8 rows 30 us against 33 us there, but 4096 -> 4096 and 11008 -> 4096 are well ahead on the GEMM.
constexpr int PREFILL_MIN_ROWS = 8;
constexpr int PREFILL_CHUNK_ROWS = 4096;  // rows per GEMM call (bounds the workspace)

std::mutex g_mu;
std::map<CacheKey, cq_layer> g_cache;
std::map<CacheKey, cq_tlayer> g_tcache;
std::map<CacheKey, cq_rlayer> g_rcache;
std::map<int, DeviceState> g_dev;

int device_state(int dev, DeviceState* out) {
  auto it = g_dev.find(dev);
  if (it == g_dev.end()) {
    DeviceState ds;
    CQ_CUDA_TRY(cudaMalloc(&ds.scratch, cq_scratch_bytes()));
    CQ_CUDA_TRY(cudaMemset(ds.scratch, 0, cq_scratch_bytes()));
    CQ_CUDA_TRY(cudaMalloc((void**)&ds.status, 256));
    CQ_CUDA_TRY(cudaMemset(ds.status, 0, 256));
    it = g_dev.emplace(dev, ds).first;
  }
  *out = it->second;
  return CQ_OK;
}

// Prefill: y += x . W^T through the tile-layout copy of the layer and the tcgen05 GEMM.
int legacy_gemm(const CacheKey& key, int dev, const void* vec, const uint8_t* qweight, const void* cherry_weight,
                const int16_t* cherry_indices, const void* scales, void* mul, int batch, uint32_t* status,
                cudaStream_t st) {
  auto it = g_tcache.find(key);
  if (it == g_tcache.end()) {
    cq_tlayer L;
    int rc = cq_tlayer_init(&L, key.bits, key.K, key.N, key.C, key.G, nullptr);
    if (rc) return rc;
    void* blob = nullptr;
    CQ_CUDA_TRY(cudaMalloc(&blob, L.blob_bytes));
    L.blob = blob;
    rc = cq_tlayer_prepare(&L, qweight, scales, cherry_weight, cherry_indices, st);
    if (rc) {
      cudaFree(blob);
      return rc;
    }
    it = g_tcache.emplace(key, L).first;
  }
  const cq_tlayer& L = it->second;
  DeviceState& ds = g_dev[dev];
  const int chunk = batch < PREFILL_CHUNK_ROWS ? batch : PREFILL_CHUNK_ROWS;
  const size_t need = cq_tlayer_gemm_workspace_bytes(&L, chunk);
  if (need > ds.gemm_ws_bytes) {
    if (ds.gemm_ws) {
      CQ_CUDA_TRY(cudaStreamSynchronize(st));   // earlier GEMMs may still read the old buffer
      CQ_CUDA_TRY(cudaFree(ds.gemm_ws));
      ds.gemm_ws = nullptr;
      ds.gemm_ws_bytes = 0;
    }
    CQ_CUDA_TRY(cudaMalloc(&ds.gemm_ws, need));
    ds.gemm_ws_bytes = need;
  }
  const __half* xp = (const __half*)vec;
  __half* yp = (__half*)mul;
  for (int m0 = 0; m0 < batch; m0 += PREFILL_CHUNK_ROWS) {
    const int rows = batch - m0 < PREFILL_CHUNK_ROWS ? batch - m0 : PREFILL_CHUNK_ROWS;
    const int rc = cq_tlayer_gemm(&L, xp + (size_t)m0 * key.K, key.K, yp + (size_t)m0 * key.N, key.N, rows,
                                  /*accumulate=*/1, ds.gemm_ws, status, st);
    if (rc) return rc;
  }
  return CQ_OK;
}

int legacy_matmul(int bits, const void* vec, const uint8_t* qweight, const void* cherry_weight,
                  const int16_t* cherry_indices, const void* scales, void* mul, int batch, int vec_height,
                  int height, int width, int cherry_size, int group_size, uint64_t tag, cudaStream_t st) {
  if (!vec || !qweight || !scales || !mul) return CQ_ERR_BAD_ARG;
  if (batch < 1) return CQ_ERR_BAD_ARG;
  if (group_size == -1) group_size = vec_height;
  const int Kc = vec_height - cherry_size;
  if (Kc <= 0 || Kc % 8 || height != Kc / 8 * bits) return CQ_ERR_BAD_SHAPE;
  int dev = 0;
  CQ_CUDA_TRY(cudaGetDevice(&dev));

  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState ds;
  int rc = device_state(dev, &ds);
  if (rc) return rc;
  const CacheKey key{dev, qweight, scales, cherry_weight, cherry_indices, bits, vec_height, width,
                     cherry_size, group_size, tag};
  // decode batches: the row-tile kernel (four activation rows per launch) up to the batch where the tile
  // GEMM overtakes it (12 rows, 8 for layers split along K); layers the row kernel does not take: the stream kernel
  // below 8 rows
  int row_limit = PREFILL_MIN_ROWS - 1;
  {
    cq_rlayer probe;
    if (cq_rlayer_init(&probe, bits, vec_height, width, cherry_size, group_size, nullptr) == CQ_OK) {
      const int pr = cq_rlayer_preferred_rows(&probe);
      if (pr > 0) row_limit = pr;
    }
  }
  if (batch > row_limit)
    return legacy_gemm(key, dev, vec, qweight, cherry_weight, cherry_indices, scales, mul, batch, ds.status, st);
  {
    auto rit = g_rcache.find(key);
    if (rit == g_rcache.end()) {
      cq_rlayer R;
      rc = cq_rlayer_init(&R, bits, vec_height, width, cherry_size, group_size, nullptr);
      if (rc == CQ_OK) rc = cq_rlayer_check(&R);
      if (rc == CQ_OK) {
        void* blob = nullptr;
        CQ_CUDA_TRY(cudaMalloc(&blob, R.blob_bytes));
        R.blob = blob;
        rc = cq_rlayer_prepare(&R, qweight, scales, cherry_weight, cherry_indices, st);
        if (rc) {
          cudaFree(blob);
          return rc;
        }
        // the kernel copies weights ahead of stream order: finish the re-pack first
        CQ_CUDA_TRY(cudaStreamSynchronize(st));
        rit = g_rcache.emplace(key, R).first;
      } else if (rc != CQ_ERR_UNSUPPORTED && rc != CQ_ERR_TOO_LARGE) {
        return rc;
      }
    }
    if (rit != g_rcache.end())
    {
      const cq_rlayer* R = &rit->second;
      return cq_rlayers_matvec(&R, 1, vec, vec_height, &mul, width, batch, /*accumulate=*/1, ds.status, st);
    }
  }
  auto it = g_cache.find(key);
  if (it == g_cache.end()) {
    cq_layer L;
    rc = cq_layer_init(&L, bits, vec_height, width, cherry_size, group_size, nullptr);
    if (rc) return rc;
    void* blob = nullptr;
    CQ_CUDA_TRY(cudaMalloc(&blob, L.blob_bytes));
    L.blob = blob;
    rc = cq_layer_prepare(&L, qweight, scales, cherry_weight, cherry_indices, st);
    if (rc) {
      cudaFree(blob);
      return rc;
    }
    // The matvec prefetches weights before it waits for the previous kernel in the
    // stream; make the freshly written stream visible first.
    CQ_CUDA_TRY(cudaStreamSynchronize(st));
    it = g_cache.emplace(key, L).first;
  }
  return cq_layer_matvec(&it->second, vec, vec_height, mul, width, batch, /*accumulate=*/1, ds.scratch,
                         ds.status, st);
}

}  // namespace

void cq_set_cuda_error(int err) { g_last_cuda_error = err; }

extern "C" int cq_last_cuda_error(void) { return g_last_cuda_error; }
extern "C" int cq_abi_version(void) { return 3; }

extern "C" const char* cq_strerror(int status) {
  switch (status) {
    case CQ_OK: return "ok";
    case CQ_ERR_BAD_ARG: return "bad argument (null or misaligned pointer, or negative size)";
    case CQ_ERR_BAD_BITS: return "bits must be 3 or 4";
    case CQ_ERR_BAD_GROUP: return "`group_size` must be 64 or a multiple of 128";
    case CQ_ERR_BAD_SHAPE: return "inconsistent layer shape";
    case CQ_ERR_TOO_LARGE: return "layer does not fit the kernel's shared-memory plan";
    case CQ_ERR_CUDA: return "CUDA runtime error";
    case CQ_ERR_NO_DEVICE: return "no usable CUDA device";
    case CQ_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
    case CQ_ERR_UNSUPPORTED: return "not supported by this build";
    case CQ_ERR_STATIC_LIMIT:
      return "request exceeds the built-in scratch of cq_layer_matvec_static (more than 16 rows, more "
             "than 256 SMs, or a layer whose rows do not fit one launch); use cq_layer_matvec";
    default: return "unknown status";
  }
}

extern "C" int cq_vecquant4matmul_cherryq(const void* vec, const uint8_t* qweight, const void* cherry_weight,
                                          const int16_t* cherry_indices, const void* scaling_factors,
                                          void* mul, int batch, int vec_height, int height, int width,
                                          int cherry_size, int group_size, uint64_t version_tag,
                                          cq_stream_t stream) {
  // csrc/quant_cuda_kernel.cu:684 of the reference rejects group sizes below 128 for 4-bit.
  if (group_size != -1 && group_size < 128) return CQ_ERR_BAD_GROUP;
  return legacy_matmul(4, vec, qweight, cherry_weight, cherry_indices, scaling_factors, mul, batch,
                       vec_height, height, width, cherry_size, group_size, version_tag,
                       (cudaStream_t)stream);
}

extern "C" int cq_vecquant3matmul_cherryq(const void* vec, const uint8_t* qweight, const void* cherry_weight,
                                          const void* cherry_indices, const void* scaling_factors, void* mul,
                                          int batch, int vec_height, int height, int width, int cherry_size,
                                          int group_size, int fp16, uint64_t version_tag,
                                          cq_stream_t stream) {
  if (group_size == -1) group_size = vec_height;
  // The reference launches nothing for other group sizes (csrc/quant_cuda_kernel.cu:139-179);
  // an error is returned instead of silently leaving `mul` untouched.
  if (!(group_size == 64 || (group_size > 0 && group_size % 128 == 0))) return CQ_ERR_BAD_GROUP;
  if (fp16)
    return legacy_matmul(3, vec, qweight, cherry_weight, (const int16_t*)cherry_indices, scaling_factors,
                         mul, batch, vec_height, height, width, cherry_size, group_size, version_tag,
                         (cudaStream_t)stream);
  if (!vec || !qweight || !scaling_factors || !mul || batch < 1) return CQ_ERR_BAD_ARG;
  const int Kc = vec_height - cherry_size;
  if (Kc <= 0 || Kc % 8 || height != Kc / 8 * 3 || width <= 0) return CQ_ERR_BAD_SHAPE;
  return cq_launch_matvec_f32(3, (const float*)vec, qweight, (const float*)cherry_weight,
                              (const int32_t*)cherry_indices, (const float*)scaling_factors, (float*)mul,
                              batch, vec_height, width, cherry_size, group_size, (cudaStream_t)stream);
}

extern "C" int cq_cache_clear(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  cudaDeviceSynchronize();
  for (auto& kv : g_cache) {
    int cur = 0;
    cudaGetDevice(&cur);
    if (cur != kv.first.dev) cudaSetDevice(kv.first.dev);
    cudaFree(kv.second.blob);
    if (cur != kv.first.dev) cudaSetDevice(cur);
  }
  g_cache.clear();
  for (auto& kv : g_tcache) {
    int cur = 0;
    cudaGetDevice(&cur);
    if (cur != kv.first.dev) cudaSetDevice(kv.first.dev);
    cudaFree(kv.second.blob);
    if (cur != kv.first.dev) cudaSetDevice(cur);
  }
  g_tcache.clear();
  for (auto& kv : g_rcache) {
    int cur = 0;
    cudaGetDevice(&cur);
    if (cur != kv.first.dev) cudaSetDevice(kv.first.dev);
    cudaFree(kv.second.blob);
    if (cur != kv.first.dev) cudaSetDevice(cur);
  }
  g_rcache.clear();
  return CQ_OK;
}

// Drops every cached copy made from this set of buffer addresses on the current device
// (any dimensions, any tag).  Synchronises the device first: a launch may still read a copy.
extern "C" int cq_cache_evict(const void* qweight, const void* scales, const void* cherry_weight,
                              const void* cherry_indices) {
  int dev = 0;
  CQ_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_mu);
  auto match = [&](const CacheKey& k) {
    return k.dev == dev && k.q == qweight && k.s == scales && k.cw == cherry_weight && k.idx == cherry_indices;
  };
  bool synced = false;
  auto drop = [&](auto& cache) {
    for (auto it = cache.begin(); it != cache.end();) {
      if (match(it->first)) {
        if (!synced) { cudaDeviceSynchronize(); synced = true; }
        cudaFree(it->second.blob);
        it = cache.erase(it);
      } else {
        ++it;
      }
    }
  };
  drop(g_cache);
  drop(g_tcache);
  drop(g_rcache);
  return CQ_OK;
}

extern "C" int cq_cache_stats(int* n_layers, uint64_t* bytes) {
  std::lock_guard<std::mutex> lock(g_mu);
  uint64_t b = 0;
  for (auto& kv : g_cache) b += kv.second.blob_bytes;
  for (auto& kv : g_tcache) b += kv.second.blob_bytes;
  for (auto& kv : g_rcache) b += kv.second.blob_bytes;
  if (n_layers) *n_layers = (int)(g_cache.size() + g_tcache.size() + g_rcache.size());
  if (bytes) *bytes = b;
  return CQ_OK;
}

extern "C" int cq_poll(cq_stream_t stream) {
  int dev = 0;
  CQ_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_dev.find(dev);
  if (it == g_dev.end()) return CQ_OK;
  uint32_t word = 0;
  CQ_CUDA_TRY(cudaMemcpyAsync(&word, it->second.status, sizeof(word), cudaMemcpyDeviceToHost,
                              (cudaStream_t)stream));
  CQ_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
  if (word == 0) return CQ_OK;
  // a timed-out launch may have left cross-CTA flags behind: start clean
  CQ_CUDA_TRY(cudaMemsetAsync(it->second.status, 0, sizeof(word), (cudaStream_t)stream));
  CQ_CUDA_TRY(cudaMemsetAsync(it->second.scratch, 0, cq_scratch_bytes(), (cudaStream_t)stream));
  CQ_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
  return CQ_ERR_DEVICE_TIMEOUT;
}
