// Python module `quant_cuda`: same name, function names, argument order and dtypes as
// the reference's extension (csrc/quant_cuda.cpp:41-77 of the reference project), so
// that llama/qlinear.py and benchmark_speed.py of the reference run against it
// unchanged.  This file holds no device code: it validates the tensors, picks the
// current CUDA stream and device, and calls the C ABI declared in include/cherryq.h.
// Differences from the reference, all deliberate:
//   * work is enqueued on torch's CURRENT stream (the reference uses the legacy
//     default stream), so the ops can be captured in CUDA graphs;
//   * a device guard covers all four ops (the reference guards only the matmuls);
//   * wrong dtypes / devices / shapes / group sizes raise RuntimeError (the
//     reference's 3-bit op silently does nothing for an unsupported group size).
// The first matmul call with a given set of weight tensors re-packs them on the GPU
// (allocates and synchronises), so it must happen before any stream capture.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>
#include <cmath>

#include <array>
#include <map>
#include <mutex>
#include <vector>

#include "cherryq.h"

namespace {

void check_status(int rc, const char* what) {
  if (rc == CQ_OK) return;
  if (rc == CQ_ERR_CUDA) {
    TORCH_CHECK(false, what, ": CUDA error ", cq_last_cuda_error());
  }
  TORCH_CHECK(false, what, ": ", cq_strerror(rc));
}

void check_tensor(const torch::Tensor& t, const char* name, c10::ScalarType dtype, const torch::Tensor& like) {
  TORCH_CHECK(t.defined(), name, " is undefined");
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == dtype, name, " must have dtype ", c10::toString(dtype), ", got ",
              c10::toString(t.scalar_type()));
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.device() == like.device(), name, " is on ", t.device(), " but vec is on ", like.device());
}

cq_stream_t current_stream() { return (cq_stream_t)c10::cuda::getCurrentCUDAStream().stream(); }

// The C library caches re-packed copies by buffer ADDRESS.  Torch's allocator hands a freed block to
// the next tensor of the same size, so an address alone does not identify a buffer: every cached set
// is paired here with weak references to the four tensors' storages.  A call whose storages are not
// the ones on record (or whose record has expired) evicts the library's copies for these addresses
// before it proceeds, and every such miss also sweeps the records whose storages have died, which
// frees their copies.  The reference's ops keep no state at all (csrc/quant_cuda.cpp:56-69).
struct StorageGuard {
  std::vector<c10::weak_intrusive_ptr<c10::StorageImpl>> w;   // four entries
  const void* ptr[4];
  int device;
};
std::mutex g_guard_mu;
std::map<std::array<const void*, 4>, StorageGuard> g_guards;

void guard_buffers(const torch::Tensor& q, const torch::Tensor& s, const torch::Tensor& cw, const torch::Tensor& ci) {
  const torch::Tensor* t[4] = {&q, &s, &cw, &ci};
  std::array<const void*, 4> key = {q.data_ptr(), s.data_ptr(), cw.data_ptr(), ci.data_ptr()};
  std::lock_guard<std::mutex> lock(g_guard_mu);
  auto it = g_guards.find(key);
  if (it != g_guards.end()) {
    bool same = true;
    for (int i = 0; i < 4; ++i) {
      auto sp = it->second.w[i].lock();
      same = same && sp && sp.get() == t[i]->storage().unsafeGetStorageImpl();
    }
    if (same) return;
    g_guards.erase(it);
  }
  // unknown or recycled addresses: whatever the library holds for them is stale
  cq_cache_evict(key[0], key[1], key[2], key[3]);
  for (auto g = g_guards.begin(); g != g_guards.end();) {
    bool dead = false;
    for (int i = 0; i < 4; ++i) dead = dead || g->second.w[i].expired();
    if (dead) {
      const at::cuda::OptionalCUDAGuard dg(c10::Device(c10::kCUDA, (c10::DeviceIndex)g->second.device));
      cq_cache_evict(g->second.ptr[0], g->second.ptr[1], g->second.ptr[2], g->second.ptr[3]);
      g = g_guards.erase(g);
    } else {
      ++g;
    }
  }
  StorageGuard ng;
  for (int i = 0; i < 4; ++i) {
    ng.w.push_back(t[i]->storage().getWeakStorageImpl());
    ng.ptr[i] = key[i];
  }
  ng.device = q.device().index();
  g_guards.emplace(key, std::move(ng));
}

uint64_t version_tag(const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& c,
                     const torch::Tensor& d) {
  // inference tensors (created under torch.inference_mode) keep no version counter
  auto v = [](const torch::Tensor& t) -> uint64_t { return t.is_inference() ? 0u : (uint64_t)t._version(); };
  return v(a) + (v(b) << 16) + (v(c) << 32) + (v(d) << 48);
}

void vecquant3matmul_cherryq(torch::Tensor vec, torch::Tensor qweight, torch::Tensor cherry_weight,
                             torch::Tensor cherry_indices, torch::Tensor scaling_factors, torch::Tensor mul,
                             int group_size, bool fp16) {
  const at::cuda::OptionalCUDAGuard device_guard(device_of(vec));
  const auto ft = fp16 ? torch::kFloat16 : torch::kFloat32;
  const auto it = fp16 ? torch::kInt16 : torch::kInt32;
  check_tensor(vec, "vec", ft, vec);
  check_tensor(qweight, "qweight", torch::kUInt8, vec);
  check_tensor(cherry_weight, "cherry_weight", ft, vec);
  check_tensor(cherry_indices, "cherry_indices", it, vec);
  check_tensor(scaling_factors, "scaling_factors", ft, vec);
  check_tensor(mul, "mul", ft, vec);
  TORCH_CHECK(vec.dim() == 2 && qweight.dim() == 2 && mul.dim() == 2, "vec, qweight and mul must be 2-D");
  TORCH_CHECK(mul.size(0) == vec.size(0) && mul.size(1) == qweight.size(1), "mul must be (batch, width)");
  TORCH_CHECK(cherry_weight.numel() == cherry_indices.size(0) * qweight.size(1), "cherry_weight must be (C, width)");
  if (fp16) guard_buffers(qweight, scaling_factors, cherry_weight, cherry_indices);
  check_status(cq_vecquant3matmul_cherryq(
                   vec.data_ptr(), qweight.data_ptr<uint8_t>(), cherry_weight.data_ptr(), cherry_indices.data_ptr(),
                   scaling_factors.data_ptr(), mul.data_ptr(), (int)vec.size(0), (int)vec.size(1),
                   (int)qweight.size(0), (int)qweight.size(1), (int)cherry_indices.size(0), group_size, fp16 ? 1 : 0,
                   version_tag(qweight, cherry_weight, cherry_indices, scaling_factors), current_stream()),
               "vecquant3matmul_cherryq");
}

void vecquant4matmul_cherryq(torch::Tensor vec, torch::Tensor qweight, torch::Tensor cherry_weight,
                             torch::Tensor cherry_indices, torch::Tensor scaling_factors, torch::Tensor mul,
                             int group_size) {
  const at::cuda::OptionalCUDAGuard device_guard(device_of(vec));
  check_tensor(vec, "vec", torch::kFloat16, vec);
  check_tensor(qweight, "qweight", torch::kUInt8, vec);
  check_tensor(cherry_weight, "cherry_weight", torch::kFloat16, vec);
  check_tensor(cherry_indices, "cherry_indices", torch::kInt16, vec);
  check_tensor(scaling_factors, "scaling_factors", torch::kFloat16, vec);
  check_tensor(mul, "mul", torch::kFloat16, vec);
  TORCH_CHECK(vec.dim() == 2 && qweight.dim() == 2 && mul.dim() == 2, "vec, qweight and mul must be 2-D");
  TORCH_CHECK(mul.size(0) == vec.size(0) && mul.size(1) == qweight.size(1), "mul must be (batch, width)");
  TORCH_CHECK(cherry_weight.numel() == cherry_indices.size(0) * qweight.size(1), "cherry_weight must be (C, width)");
  guard_buffers(qweight, scaling_factors, cherry_weight, cherry_indices);
  check_status(cq_vecquant4matmul_cherryq(
                   vec.data_ptr(), qweight.data_ptr<uint8_t>(), cherry_weight.data_ptr(),
                   (const int16_t*)cherry_indices.data_ptr(), scaling_factors.data_ptr(), mul.data_ptr(),
                   (int)vec.size(0), (int)vec.size(1), (int)qweight.size(0), (int)qweight.size(1),
                   (int)cherry_indices.size(0), group_size,
                   version_tag(qweight, cherry_weight, cherry_indices, scaling_factors), current_stream()),
               "vecquant4matmul_cherryq");
}

void dequantize_normal(int bits, torch::Tensor qweight, torch::Tensor scaling_factors, torch::Tensor out, int height,
                       int cherry_size, int group_size) {
  const at::cuda::OptionalCUDAGuard device_guard(device_of(qweight));
  check_tensor(qweight, "qweight", torch::kUInt8, qweight);
  check_tensor(scaling_factors, "scaling_factors", torch::kFloat32, qweight);
  check_tensor(out, "out", torch::kFloat32, qweight);
  TORCH_CHECK(qweight.dim() == 2 && out.dim() == 2 && out.size(1) == qweight.size(1) &&
                  out.size(0) >= height - cherry_size,
              "out must be (>= height - cherry_size, width)");
  auto fn = bits == 3 ? cq_dequantize3_normal : cq_dequantize4_normal;
  check_status(fn(qweight.data_ptr<uint8_t>(), scaling_factors.data_ptr<float>(), out.data_ptr<float>(),
                  (int)qweight.size(0), (int)qweight.size(1), height, cherry_size, group_size, current_stream()),
               bits == 3 ? "Dequantize3Normal" : "Dequantize4Normal");
}

void Dequantize3Normal(torch::Tensor qweight, torch::Tensor scaling_factors, torch::Tensor out, int height,
                       int cherry_size, int group_size) {
  dequantize_normal(3, qweight, scaling_factors, out, height, cherry_size, group_size);
}
void Dequantize4Normal(torch::Tensor qweight, torch::Tensor scaling_factors, torch::Tensor out, int height,
                       int cherry_size, int group_size) {
  dequantize_normal(4, qweight, scaling_factors, out, height, cherry_size, group_size);
}

// ------------------------------------------------------------------ additive entry points
// GPU QuantLinear.pack (llama/qlinear.py:67-118): returns (qweight, scales, cherry_weight, cherry_indices).
std::vector<torch::Tensor> pack(torch::Tensor weight, torch::Tensor cherry_unsorted, int bits, int group_size) {
  const at::cuda::OptionalCUDAGuard device_guard(device_of(weight));
  TORCH_CHECK(weight.is_cuda() && weight.dim() == 2 && weight.is_contiguous(), "weight must be a contiguous 2-D CUDA tensor");
  TORCH_CHECK(weight.scalar_type() == torch::kFloat16 || weight.scalar_type() == torch::kFloat32,
              "weight must be float16 or float32");
  check_tensor(cherry_unsorted, "cherry_indices", torch::kInt32, weight);
  const int N = (int)weight.size(0), K = (int)weight.size(1), C = (int)cherry_unsorted.numel();
  const int G = group_size == -1 ? K : group_size;
  TORCH_CHECK(G > 0, "group_size must be positive or -1");
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0 && C % 8 == 0 && C < K, "in_features, out_features and the cherry count must be multiples of 8");
  auto u8 = torch::TensorOptions().device(weight.device()).dtype(torch::kUInt8);
  auto qweight = torch::empty({(K - C) / 8 * bits, N}, u8);
  auto scales = torch::empty({(K - C + G - 1) / G, N}, u8.dtype(torch::kFloat16));
  auto cw = torch::empty({C, N}, u8.dtype(torch::kFloat16));
  auto idx = torch::empty({C}, u8.dtype(torch::kInt16));
  check_status(cq_pack(weight.data_ptr(), weight.scalar_type() == torch::kFloat32, cherry_unsorted.data_ptr<int32_t>(),
                       bits, K, N, C, G, qweight.data_ptr<uint8_t>(), scales.data_ptr(), cw.data_ptr(),
                       (int16_t*)idx.data_ptr(), nullptr, current_stream()),
               "pack");
  return {qweight, scales, cw, idx};
}

// GPU QuantLinear.unpack (llama/qlinear.py:120-162): dense (N, K) fp16.
torch::Tensor unpack_dense(torch::Tensor qweight, torch::Tensor scales, torch::Tensor cherry_weight,
                           torch::Tensor cherry_indices, int bits, int in_features, int group_size) {
  const at::cuda::OptionalCUDAGuard device_guard(device_of(qweight));
  check_tensor(qweight, "qweight", torch::kUInt8, qweight);
  check_tensor(scales, "scales", torch::kFloat16, qweight);
  check_tensor(cherry_weight, "cherry_weight", torch::kFloat16, qweight);
  check_tensor(cherry_indices, "cherry_indices", torch::kInt16, qweight);
  const int N = (int)qweight.size(1), C = (int)cherry_indices.numel();
  auto dense = torch::empty({N, in_features}, scales.options());
  check_status(cq_unpack_dense(qweight.data_ptr<uint8_t>(), scales.data_ptr(), cherry_weight.data_ptr(),
                               (const int16_t*)cherry_indices.data_ptr(), bits, in_features, N, C, group_size,
                               dense.data_ptr(), current_stream()),
               "unpack_dense");
  return dense;
}

std::mutex g_mu;
std::map<int, torch::Tensor> g_scratch;  // per device: matvec scratch followed by a status word
std::map<int, torch::Tensor> g_attn_ws;  // per device: workspace of the decode attention

torch::Tensor scratch_for(const torch::Device& dev) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_scratch.find(dev.index());
  if (it == g_scratch.end()) {
    auto t = torch::zeros({(int64_t)cq_scratch_bytes() + 256}, torch::TensorOptions().device(dev).dtype(torch::kUInt8));
    it = g_scratch.emplace(dev.index(), t).first;
  }
  return it->second;
}

// A layer re-packed into the stream layout; owns its device blob.
struct PreparedLayer {
  cq_layer layer;
  torch::Tensor blob;

  PreparedLayer(torch::Tensor qweight, torch::Tensor scales, torch::Tensor cherry_weight,
                torch::Tensor cherry_indices, int bits, int in_features, int group_size) {
    const at::cuda::OptionalCUDAGuard device_guard(device_of(qweight));
    check_tensor(qweight, "qweight", torch::kUInt8, qweight);
    check_tensor(scales, "scales", torch::kFloat16, qweight);
    check_tensor(cherry_weight, "cherry_weight", torch::kFloat16, qweight);
    check_tensor(cherry_indices, "cherry_indices", torch::kInt16, qweight);
    const int N = (int)qweight.size(1), C = (int)cherry_indices.numel();
    check_status(cq_layer_init(&layer, bits, in_features, N, C, group_size, nullptr), "PreparedLayer");
    TORCH_CHECK(qweight.size(0) == layer.Kc / 8 * bits, "qweight has ", qweight.size(0), " rows, expected ",
                layer.Kc / 8 * bits);
    TORCH_CHECK(scales.size(0) == (layer.Kc + layer.G - 1) / layer.G && scales.size(1) == N, "scales must be (ceil(K'/G), N)");
    blob = torch::empty({(int64_t)layer.blob_bytes}, qweight.options());
    layer.blob = blob.data_ptr();
    check_status(cq_layer_prepare(&layer, qweight.data_ptr<uint8_t>(), scales.data_ptr(), cherry_weight.data_ptr(),
                                  (const int16_t*)cherry_indices.data_ptr(), current_stream()),
                 "PreparedLayer");
    // the matvec prefetches weights ahead of stream order: finish the re-pack first
    c10::cuda::getCurrentCUDAStream().synchronize();
  }

  // A layer rebuilt around an existing blob (e.g. loaded from a file or sliced from a shard).
  PreparedLayer(torch::Tensor blob_, int bits, int in_features, int out_features, int num_cherries, int group_size) {
    TORCH_CHECK(blob_.is_cuda() && blob_.scalar_type() == torch::kUInt8 && blob_.is_contiguous(), "blob must be a contiguous CUDA uint8 tensor");
    check_status(cq_layer_init(&layer, bits, in_features, out_features, num_cherries, group_size, nullptr), "PreparedLayer");
    TORCH_CHECK((uint64_t)blob_.numel() == layer.blob_bytes, "blob has ", blob_.numel(), " bytes, expected ", layer.blob_bytes);
    TORCH_CHECK(((uintptr_t)blob_.data_ptr() & 255) == 0, "blob must be 256-byte aligned");
    blob = blob_;
    layer.blob = blob.data_ptr();
  }

  // out (M, N) fp16 = [out +] x (M, K) fp16 . W^T
  void matvec(torch::Tensor x, torch::Tensor out, bool accumulate) {
    const at::cuda::OptionalCUDAGuard device_guard(device_of(x));
    check_tensor(x, "x", torch::kFloat16, blob);
    check_tensor(out, "out", torch::kFloat16, blob);
    TORCH_CHECK(x.dim() == 2 && x.size(1) == layer.K, "x must be (M, ", layer.K, ")");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == x.size(0) && out.size(1) == layer.N, "out must be (M, ", layer.N, ")");
    auto scratch = scratch_for(x.device());
    uint8_t* sp = scratch.data_ptr<uint8_t>();
    check_status(cq_layer_matvec(&layer, x.data_ptr(), layer.K, out.data_ptr(), layer.N, (int)x.size(0),
                                 accumulate ? 1 : 0, sp, (uint32_t*)(sp + cq_scratch_bytes()), current_stream()),
                 "PreparedLayer.matvec");
  }

  // Back to the reference's four buffers: (qweight, scales, cherry_weight, cherry_indices).
  std::vector<torch::Tensor> unprepare() {
    const at::cuda::OptionalCUDAGuard device_guard(device_of(blob));
    auto o = blob.options();
    auto qweight = torch::empty({layer.Kc / 8 * layer.bits, layer.N}, o);
    auto scales = torch::empty({(layer.Kc + layer.G - 1) / layer.G, layer.N}, o.dtype(torch::kFloat16));
    auto cw = torch::empty({layer.C, layer.N}, o.dtype(torch::kFloat16));
    auto idx = torch::empty({layer.C}, o.dtype(torch::kInt16));
    check_status(cq_layer_unprepare(&layer, qweight.data_ptr<uint8_t>(), scales.data_ptr(), cw.data_ptr(),
                                    (int16_t*)idx.data_ptr(), current_stream()),
                 "PreparedLayer.unprepare");
    return {qweight, scales, cw, idx};
  }
};

// A layer re-packed into the row-tile layout of the one-row decode kernel; owns its device blob.
struct RowLayer {
  cq_rlayer layer;
  torch::Tensor blob;

  // CQ_OK if the one-row kernel can run such a layer on the current device
  static bool supported(int bits, int in_features, int out_features, int num_cherries, int group_size) {
    cq_rlayer L;
    if (cq_rlayer_init(&L, bits, in_features, out_features, num_cherries, group_size, nullptr) != CQ_OK) return false;
    return cq_rlayer_check(&L) == CQ_OK;
  }

  RowLayer(torch::Tensor qweight, torch::Tensor scales, torch::Tensor cherry_weight, torch::Tensor cherry_indices,
           int bits, int in_features, int group_size) {
    const at::cuda::OptionalCUDAGuard device_guard(device_of(qweight));
    check_tensor(qweight, "qweight", torch::kUInt8, qweight);
    check_tensor(scales, "scales", torch::kFloat16, qweight);
    check_tensor(cherry_weight, "cherry_weight", torch::kFloat16, qweight);
    check_tensor(cherry_indices, "cherry_indices", torch::kInt16, qweight);
    const int N = (int)qweight.size(1), C = (int)cherry_indices.numel();
    check_status(cq_rlayer_init(&layer, bits, in_features, N, C, group_size, nullptr), "RowLayer");
    check_status(cq_rlayer_check(&layer), "RowLayer");
    TORCH_CHECK(qweight.size(0) == layer.Kc / 8 * bits, "qweight has ", qweight.size(0), " rows, expected ",
                layer.Kc / 8 * bits);
    TORCH_CHECK(scales.size(0) == (layer.Kc + layer.G - 1) / layer.G && scales.size(1) == N, "scales must be (ceil(K'/G), N)");
    blob = torch::empty({(int64_t)layer.blob_bytes}, qweight.options());
    layer.blob = blob.data_ptr();
    check_status(cq_rlayer_prepare(&layer, qweight.data_ptr<uint8_t>(), scales.data_ptr(), cherry_weight.data_ptr(),
                                   (const int16_t*)cherry_indices.data_ptr(), current_stream()),
                 "RowLayer");
    // the kernel copies weights ahead of stream order: finish the re-pack first
    c10::cuda::getCurrentCUDAStream().synchronize();
  }

  // out (M, N) fp16 = [out +] x (M, K) fp16 . W^T; four rows per launch
  void matvec(torch::Tensor x, torch::Tensor out, bool accumulate) {
    const at::cuda::OptionalCUDAGuard device_guard(device_of(x));
    check_tensor(x, "x", torch::kFloat16, blob);
    check_tensor(out, "out", torch::kFloat16, blob);
    TORCH_CHECK(x.numel() % layer.K == 0 && x.numel() > 0, "x must hold rows of ", layer.K, " activations");
    const int M = (int)(x.numel() / layer.K);
    TORCH_CHECK(out.numel() == (int64_t)M * layer.N, "out must hold ", M, " rows of ", layer.N, " values");
    auto scratch = scratch_for(x.device());
    uint8_t* sp = scratch.data_ptr<uint8_t>();
    const cq_rlayer* lp = &layer;
    void* yp = out.data_ptr();
    check_status(cq_rlayers_matvec(&lp, 1, x.data_ptr(), layer.K, &yp, layer.N, M, accumulate ? 1 : 0,
                                   (uint32_t*)(sp + cq_scratch_bytes()), current_stream()),
                 "RowLayer.matvec");
  }

  // out (M, N) fp16 = (silu(gate) * up) (M, K) . W^T: the SwiGLU of a gated MLP folded into the down projection
  void matvec_swiglu(torch::Tensor gate, torch::Tensor up, torch::Tensor out) {
    const at::cuda::OptionalCUDAGuard device_guard(device_of(gate));
    check_tensor(gate, "gate", torch::kFloat16, blob);
    check_tensor(up, "up", torch::kFloat16, blob);
    check_tensor(out, "out", torch::kFloat16, blob);
    TORCH_CHECK(gate.sizes() == up.sizes() && gate.numel() % layer.K == 0 && gate.numel() > 0,
                "gate and up must hold the same rows of ", layer.K, " values");
    const int M = (int)(gate.numel() / layer.K);
    TORCH_CHECK(out.numel() == (int64_t)M * layer.N, "out must hold ", M, " rows of ", layer.N, " values");
    auto scratch = scratch_for(gate.device());
    uint8_t* sp = scratch.data_ptr<uint8_t>();
    check_status(cq_rlayer_matvec_swiglu(&layer, gate.data_ptr(), up.data_ptr(), layer.K, out.data_ptr(), layer.N, M,
                                         (uint32_t*)(sp + cq_scratch_bytes()), current_stream()),
                 "RowLayer.matvec_swiglu");
  }

  // Column-parallel shard: y_local (M, N) = x (M, K) . W^T and, in the same launch, the exchange of the ranks'
  // slices over peer memory: y_all (M, P * N).  regions: the P mapped region addresses (parallel.PeerAllGather).
  void matvec_gather(torch::Tensor x, torch::Tensor y_local, torch::Tensor y_all, std::vector<int64_t> regions, int rank,
                     int64_t capacity, int timeout_ms, torch::Tensor status) {
    const at::cuda::OptionalCUDAGuard device_guard(device_of(x));
    check_tensor(x, "x", torch::kFloat16, blob);
    check_tensor(y_local, "y_local", torch::kFloat16, blob);
    check_tensor(y_all, "y_all", torch::kFloat16, blob);
    check_tensor(status, "status", torch::kInt32, blob);
    TORCH_CHECK(x.numel() % layer.K == 0 && x.numel() > 0, "x must hold rows of ", layer.K, " activations");
    const int M = (int)(x.numel() / layer.K), P = (int)regions.size();
    TORCH_CHECK(y_local.numel() == (int64_t)M * layer.N && y_all.numel() == (int64_t)M * layer.N * P,
                "y_local must be (M, N) and y_all (M, P * N)");
    std::vector<void*> rp(P);
    for (int i = 0; i < P; ++i) rp[i] = (void*)(uintptr_t)regions[i];
    check_status(cq_rlayer_matvec_gather(&layer, x.data_ptr(), layer.K, y_local.data_ptr(), M, rp.data(), P, rank,
                                         (size_t)capacity, y_all.data_ptr(), timeout_ms, (uint32_t*)status.data_ptr(),
                                         current_stream()),
                 "RowLayer.matvec_gather");
  }

  // Back to the reference's four buffers: (qweight, scales, cherry_weight, cherry_indices).
  std::vector<torch::Tensor> unprepare() {
    const at::cuda::OptionalCUDAGuard device_guard(device_of(blob));
    auto o = blob.options();
    auto qweight = torch::empty({layer.Kc / 8 * layer.bits, layer.N}, o);
    auto scales = torch::empty({(layer.Kc + layer.G - 1) / layer.G, layer.N}, o.dtype(torch::kFloat16));
    auto cw = torch::empty({layer.C, layer.N}, o.dtype(torch::kFloat16));
    auto idx = torch::empty({layer.C}, o.dtype(torch::kInt16));
    check_status(cq_rlayer_unprepare(&layer, qweight.data_ptr<uint8_t>(), scales.data_ptr(), cw.data_ptr(),
                                     (int16_t*)idx.data_ptr(), current_stream()),
                 "RowLayer.unprepare");
    return {qweight, scales, cw, idx};
  }
};

// A layer re-packed into the tile layout of the tensor-core GEMM (prefill and large batches); owns its blob.
struct TileLayer {
  cq_tlayer layer;
  torch::Tensor blob;

  TileLayer(torch::Tensor qweight, torch::Tensor scales, torch::Tensor cherry_weight, torch::Tensor cherry_indices,
            int bits, int in_features, int group_size) {
    const at::cuda::OptionalCUDAGuard device_guard(device_of(qweight));
    check_tensor(qweight, "qweight", torch::kUInt8, qweight);
    check_tensor(scales, "scales", torch::kFloat16, qweight);
    check_tensor(cherry_weight, "cherry_weight", torch::kFloat16, qweight);
    check_tensor(cherry_indices, "cherry_indices", torch::kInt16, qweight);
    const int N = (int)qweight.size(1), C = (int)cherry_indices.numel();
    check_status(cq_tlayer_init(&layer, bits, in_features, N, C, group_size, nullptr), "TileLayer");
    TORCH_CHECK(qweight.size(0) == (in_features - C) / 8 * bits, "qweight has ", qweight.size(0), " rows, expected ",
                (in_features - C) / 8 * bits);
    blob = torch::empty({(int64_t)layer.blob_bytes}, qweight.options());
    layer.blob = blob.data_ptr();
    check_status(cq_tlayer_prepare(&layer, qweight.data_ptr<uint8_t>(), scales.data_ptr(), cherry_weight.data_ptr(),
                                   (const int16_t*)cherry_indices.data_ptr(), current_stream()),
                 "TileLayer");
  }

  // out (M, N) fp16 = [out +] x (M, K) fp16 . W^T, walked in slices of 4096 rows (bounds the workspace)
  void gemm(torch::Tensor x, torch::Tensor out, bool accumulate) {
    const at::cuda::OptionalCUDAGuard device_guard(device_of(x));
    check_tensor(x, "x", torch::kFloat16, blob);
    check_tensor(out, "out", torch::kFloat16, blob);
    TORCH_CHECK(x.dim() == 2 && x.size(1) == layer.K, "x must be (M, ", layer.K, ")");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == x.size(0) && out.size(1) == layer.N, "out must be (M, ", layer.N, ")");
    const int M = (int)x.size(0), CH = 4096;
    const int chunk = M < CH ? M : CH;
    auto ws = torch::empty({(int64_t)cq_tlayer_gemm_workspace_bytes(&layer, chunk)}, blob.options());
    auto scratch = scratch_for(x.device());
    uint8_t* sp = scratch.data_ptr<uint8_t>();
    const uint16_t* xp = (const uint16_t*)x.data_ptr();      // fp16 elements
    uint16_t* yp = (uint16_t*)out.data_ptr();
    for (int m0 = 0; m0 < M; m0 += CH) {
      const int rows = M - m0 < CH ? M - m0 : CH;
      check_status(cq_tlayer_gemm(&layer, xp + (size_t)m0 * layer.K, layer.K, yp + (size_t)m0 * layer.N, layer.N, rows,
                                  accumulate ? 1 : 0, ws.data_ptr(), (uint32_t*)(sp + cq_scratch_bytes()), current_stream()),
                   "TileLayer.gemm");
    }
  }
};

// One launch (per four activation rows) for several row-tile layers that take the same activations
// (q / k / v, gate / up): outs[i] = [outs[i] +] x (M, K) fp16 . W_i^T.  The outputs are rows of `ldy`
// elements each: views into one (M, ldy) buffer, or separate (M, N_i) tensors when every N_i == ldy.
void row_layers_matvec(std::vector<RowLayer*> layers, torch::Tensor x, std::vector<torch::Tensor> outs, bool accumulate) {
  TORCH_CHECK(!layers.empty() && layers.size() <= 4 && layers.size() == outs.size(), "1 to 4 layers, one output each");
  const at::cuda::OptionalCUDAGuard device_guard(device_of(x));
  check_tensor(x, "x", torch::kFloat16, layers[0]->blob);
  const int K = layers[0]->layer.K;
  TORCH_CHECK(x.numel() % K == 0 && x.numel() > 0, "x must hold rows of ", K, " activations");
  const int M = (int)(x.numel() / K);
  const cq_rlayer* ls[4];
  void* ys[4];
  int64_t ldy = -1;
  for (size_t i = 0; i < layers.size(); ++i) {
    const auto& o = outs[i];
    TORCH_CHECK(o.is_cuda() && o.scalar_type() == torch::kFloat16 && o.device() == x.device() && o.dim() == 2 &&
                o.size(0) == M && o.size(1) == layers[i]->layer.N && o.stride(1) == 1,
                "out ", i, " must be a (", M, ", ", layers[i]->layer.N, ") fp16 CUDA tensor with unit column stride");
    if (M == 1) {
      ldy = std::max<int64_t>(ldy, o.size(1));          // a single row: the stride is never used
    } else {
      TORCH_CHECK(ldy < 0 || o.stride(0) == ldy, "the outputs must share one row stride (views of one buffer)");
      ldy = o.stride(0);
    }
    ls[i] = &layers[i]->layer;
    ys[i] = o.data_ptr();
  }
  auto scratch = scratch_for(x.device());
  uint8_t* sp = scratch.data_ptr<uint8_t>();
  check_status(cq_rlayers_matvec(ls, (int)layers.size(), x.data_ptr(), K, ys, (int)ldy, M, accumulate ? 1 : 0,
                                 (uint32_t*)(sp + cq_scratch_bytes()), current_stream()),
               "row_layers_matvec");
}

// Reads and clears the status word the PreparedLayer launches report into.
bool device_timed_out(int device_index) {
  torch::Tensor t;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_scratch.find(device_index);
    if (it == g_scratch.end()) return false;
    t = it->second;
  }
  auto word = t.slice(0, (int64_t)cq_scratch_bytes(), (int64_t)cq_scratch_bytes() + 4).cpu();
  const bool bad = word.view(torch::kInt32).item<int32_t>() != 0;
  if (bad) t.zero_();
  return bad;
}

}  // namespace

// ---- element-wise kernels of the decode harness
std::vector<torch::Tensor> rmsnorm(torch::Tensor x, c10::optional<torch::Tensor> residual, torch::Tensor weight,
                                   double eps, bool return_sum) {
  const at::cuda::OptionalCUDAGuard device_guard(device_of(x));
  check_tensor(x, "x", torch::kFloat16, x);
  check_tensor(weight, "weight", torch::kFloat16, x);
  TORCH_CHECK(x.dim() == 2 && weight.numel() == x.size(1), "x must be (rows, hidden) and weight (hidden,)");
  const void* res = nullptr;
  if (residual.has_value()) {
    check_tensor(*residual, "residual", torch::kFloat16, x);
    TORCH_CHECK(residual->sizes() == x.sizes(), "residual must have the shape of x");
    res = residual->data_ptr();
  }
  auto y = torch::empty_like(x);
  torch::Tensor h;
  if (return_sum) h = torch::empty_like(x);
  check_status(cq_rmsnorm(x.data_ptr(), res, weight.data_ptr(), y.data_ptr(), return_sum ? h.data_ptr() : nullptr,
                          (int)x.size(0), (int)x.size(1), (float)eps, current_stream()),
               "rmsnorm");
  if (return_sum) return {y, h};
  return {y};
}

void rope_cache(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor cos_table, torch::Tensor sin_table,
                torch::Tensor positions, torch::Tensor k_cache, torch::Tensor v_cache) {
  const at::cuda::OptionalCUDAGuard device_guard(device_of(q));
  check_tensor(q, "q", torch::kFloat16, q);
  check_tensor(k, "k", torch::kFloat16, q);
  check_tensor(v, "v", torch::kFloat16, q);
  check_tensor(cos_table, "cos", torch::kFloat32, q);
  check_tensor(sin_table, "sin", torch::kFloat32, q);
  check_tensor(positions, "positions", torch::kInt64, q);
  check_tensor(k_cache, "k_cache", torch::kFloat16, q);
  check_tensor(v_cache, "v_cache", torch::kFloat16, q);
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.sizes() == k.sizes() && q.size(0) == k.size(0) && q.size(2) == k.size(2),
              "q must be (T, H, D), k and v (T, KV, D)");
  const int T = (int)q.size(0), H = (int)q.size(1), KV = (int)k.size(1), D = (int)q.size(2);
  TORCH_CHECK(positions.numel() == T, "positions must have T entries");
  TORCH_CHECK(cos_table.dim() == 2 && cos_table.size(1) == D / 2 && sin_table.sizes() == cos_table.sizes(),
              "cos / sin tables must be (max_seq, D / 2)");
  // caches (max_seq, KV, D): the T tokens are one sequence; (B, max_seq, KV, D): T / B consecutive tokens per sequence
  TORCH_CHECK((k_cache.dim() == 3 || k_cache.dim() == 4) && v_cache.sizes() == k_cache.sizes(), "caches must be ([B,] max_seq, KV, D)");
  const int cd = (int)k_cache.dim();
  const int B = cd == 4 ? (int)k_cache.size(0) : 1;
  TORCH_CHECK(k_cache.size(cd - 2) == KV && k_cache.size(cd - 1) == D && k_cache.size(cd - 3) <= cos_table.size(0) && T % B == 0,
              "caches must be ([B,] max_seq, KV, D) with max_seq within the rotary tables and B dividing T");
  check_status(cq_rope_cache(q.data_ptr(), k.data_ptr(), v.data_ptr(), cos_table.data_ptr<float>(),
                             sin_table.data_ptr<float>(), (const long long*)positions.data_ptr(), k_cache.data_ptr(),
                             v_cache.data_ptr(), T, H, KV, D, (int)k_cache.size(cd - 3), T / B, current_stream()),
               "rope_cache");
}

torch::Tensor silu_mul(torch::Tensor gate, torch::Tensor up) {
  const at::cuda::OptionalCUDAGuard device_guard(device_of(gate));
  check_tensor(gate, "gate", torch::kFloat16, gate);
  check_tensor(up, "up", torch::kFloat16, gate);
  TORCH_CHECK(gate.sizes() == up.sizes(), "gate and up must have the same shape");
  auto out = torch::empty_like(gate);
  check_status(cq_silu_mul(gate.data_ptr(), up.data_ptr(), out.data_ptr(), (long long)gate.numel(), current_stream()),
               "silu_mul");
  return out;
}


torch::Tensor attn_decode(torch::Tensor q, torch::Tensor k_cache, torch::Tensor v_cache, torch::Tensor position) {
  const at::cuda::OptionalCUDAGuard device_guard(device_of(q));
  check_tensor(q, "q", torch::kFloat16, q);
  check_tensor(k_cache, "k_cache", torch::kFloat16, q);
  check_tensor(v_cache, "v_cache", torch::kFloat16, q);
  check_tensor(position, "position", torch::kInt64, q);
  // q (B, H, D), one query per sequence; caches (B, max_seq, KV, D), or (max_seq, KV, D) for B == 1
  TORCH_CHECK(q.dim() == 3, "q must be (B, H, D)");
  const int B = (int)q.size(0);
  const int cd = (int)k_cache.dim();
  TORCH_CHECK((cd == 4 && k_cache.size(0) == B) || (cd == 3 && B == 1), "caches must be (B, max_seq, KV, D)");
  TORCH_CHECK(k_cache.size(cd - 1) == q.size(2) && v_cache.sizes() == k_cache.sizes(), "caches must be ([B,] max_seq, KV, D)");
  TORCH_CHECK(position.numel() == B, "one position per sequence");
  auto out = torch::empty_like(q);
  // the ranges of a head meet in a per-device workspace (grow-only, zero-filled when created; launches of one
  // stream follow one another, which is how the decode harness calls this)
  const size_t need = cq_attn_decode_workspace_bytes(B, (int)q.size(1), (int)q.size(2), (int)k_cache.size(cd - 3));
  torch::Tensor ws;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto& slot = g_attn_ws[q.device().index()];
    if (!slot.defined() || (size_t)slot.numel() < need)
      slot = torch::zeros({(int64_t)need}, torch::TensorOptions().device(q.device()).dtype(torch::kUInt8));
    ws = slot;
  }
  check_status(cq_attn_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), (const long long*)position.data_ptr(),
                              out.data_ptr(), B, (int)q.size(1), (int)k_cache.size(cd - 2), (int)q.size(2),
                              (int)k_cache.size(cd - 3), 1.0f / std::sqrt((float)q.size(2)), ws.data_ptr(), current_stream()),
               "attn_decode");
  return out;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("vecquant3matmul_cherryq", &vecquant3matmul_cherryq, "a 3-bit version");
  m.def("vecquant4matmul_cherryq", &vecquant4matmul_cherryq, "a 4-bit version");
  m.def("Dequantize3Normal", &Dequantize3Normal, "Dequantize3Normal");
  m.def("Dequantize4Normal", &Dequantize4Normal, "Dequantize4Normal");
  m.def("pack", &pack, "GPU QuantLinear.pack");
  m.def("unpack_dense", &unpack_dense, "GPU QuantLinear.unpack");
  m.def("cache_clear", []() {
    check_status(cq_cache_clear(), "cache_clear");
    std::lock_guard<std::mutex> lock(g_guard_mu);
    g_guards.clear();
  });
  m.def("cache_stats", []() {
    int n = 0;
    uint64_t b = 0;
    cq_cache_stats(&n, &b);
    return std::make_pair(n, b);
  });
  m.def("rmsnorm", &rmsnorm, "RMSNorm with optional residual add");
  m.def("rope_cache", &rope_cache, "rotary embedding in place + KV cache write");
  m.def("silu_mul", &silu_mul, "silu(gate) * up");
  m.def("attn_decode", &attn_decode, "single-query attention over the KV cache");
  m.def("poll", []() { check_status(cq_poll(current_stream()), "poll"); });
  m.def("device_timed_out", &device_timed_out);
  m.def("row_layers_matvec", &row_layers_matvec, "one launch for row-tile layers sharing an activation row");
  m.def("abi_version", &cq_abi_version);
  py::class_<RowLayer>(m, "RowLayer")
      .def(py::init<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, int, int, int>())
      .def_static("supported", &RowLayer::supported)
      .def("matvec", &RowLayer::matvec)
      .def("matvec_gather", &RowLayer::matvec_gather)
      .def("matvec_swiglu", &RowLayer::matvec_swiglu)
      .def("unprepare", &RowLayer::unprepare)
      .def_readonly("blob", &RowLayer::blob)
      .def_property_readonly("preferred_rows", [](const RowLayer& p) { return cq_rlayer_preferred_rows(&p.layer); })
      .def_property_readonly("out_features", [](const RowLayer& p) { return p.layer.N; })
      .def_property_readonly("in_features", [](const RowLayer& p) { return p.layer.K; });
  py::class_<TileLayer>(m, "TileLayer")
      .def(py::init<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, int, int, int>())
      .def("gemm", &TileLayer::gemm)
      .def_readonly("blob", &TileLayer::blob);
  py::class_<PreparedLayer>(m, "PreparedLayer")
      .def(py::init<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, int, int, int>())
      .def(py::init<torch::Tensor, int, int, int, int, int>())
      .def("matvec", &PreparedLayer::matvec)
      .def("unprepare", &PreparedLayer::unprepare)
      .def_readonly("blob", &PreparedLayer::blob)
      .def_property_readonly("bits", [](const PreparedLayer& p) { return p.layer.bits; })
      .def_property_readonly("in_features", [](const PreparedLayer& p) { return p.layer.K; })
      .def_property_readonly("out_features", [](const PreparedLayer& p) { return p.layer.N; })
      .def_property_readonly("num_cherries", [](const PreparedLayer& p) { return p.layer.C; })
      .def_property_readonly("group_size", [](const PreparedLayer& p) { return p.layer.G; });
}
