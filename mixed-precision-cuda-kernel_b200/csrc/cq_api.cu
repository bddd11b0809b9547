// extern "C" entry points that keep the reference's operator signatures
// (csrc/quant_cuda.cpp:41-69 of the reference project) on top of the prepared
// layer interface: the first call with a given set of reference buffers re-packs
// them on the GPU into the stream layout and caches the result; every call then
// runs the stream matvec.
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
};

std::mutex g_mu;
std::map<CacheKey, cq_layer> g_cache;
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
extern "C" int cq_abi_version(void) { return 1; }

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
  return CQ_OK;
}

extern "C" int cq_cache_stats(int* n_layers, uint64_t* bytes) {
  std::lock_guard<std::mutex> lock(g_mu);
  uint64_t b = 0;
  for (auto& kv : g_cache) b += kv.second.blob_bytes;
  if (n_layers) *n_layers = (int)g_cache.size();
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
