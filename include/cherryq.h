/*
 * cherryq.h — C ABI of the B200 (sm_100a) CherryQ quantized-linear library.
 *
 * Everything here is `extern "C"`, takes plain device/host pointers and sizes,
 * never throws and never aborts: every entry point returns a cq_status code
 * (0 = success) and enqueues its work on the CUDA stream it is given (pass 0
 * for the legacy default stream).  Pointers are DEVICE pointers unless a
 * parameter is documented as host memory.
 *
 * The entry points replace, one for one, the operator interface of the
 * reference project wangitu/Mixed-precision-CUDA-kernel (paths below are inside
 * that project):
 *
 *   csrc/quant_cuda.cpp:41-54   vecquant3matmul_cherryq   -> cq_vecquant3matmul_cherryq
 *   csrc/quant_cuda.cpp:56-69   vecquant4matmul_cherryq   -> cq_vecquant4matmul_cherryq
 *   csrc/quant_cuda.cpp:26-38   Dequantize3Normal / Dequantize4Normal
 *                                                         -> cq_dequantize3_normal / cq_dequantize4_normal
 *   llama/qlinear.py:67-118     QuantLinear.pack          -> cq_pack
 *   llama/qlinear.py:120-162    QuantLinear.unpack        -> cq_unpack_dense
 *
 * plus the prepared-layer interface (cq_layer_*) that the legacy calls use
 * internally: the reference's uint8 buffers are re-packed ON THE GPU into a
 * stream layout made for 16-byte shared-memory reads and tensor-core fragments,
 * and the matvec runs on that.
 *
 * Reference buffer formats (llama/qlinear.py:43-58), all row-major, N contiguous:
 *   qweight        uint8  (K'/8*bits, N)   K' = K - C compacted (cherry-free) columns
 *   scales         fp16   (ceil(K'/G), N)
 *   cherry_weight  fp16   (C, N)
 *   cherry_indices int16  (C,)  sorted ascending
 * with K = in_features, N = out_features, C = number of fp16 "cherry" columns,
 * G = group size on the compacted axis, bits in {3, 4}.
 */
#ifndef CHERRYQ_H_
#define CHERRYQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* cq_stream_t; /* a cudaStream_t */

typedef enum cq_status {
  CQ_OK = 0,
  CQ_ERR_BAD_ARG = 1,       /* null pointer, negative size, misaligned pointer            */
  CQ_ERR_BAD_BITS = 2,      /* bits is not 3 or 4                                         */
  CQ_ERR_BAD_GROUP = 3,     /* group size is not 64 or a multiple of 128                  */
  CQ_ERR_BAD_SHAPE = 4,     /* K % 8, N % 8, C % 8, K > 65534, C >= K ...                 */
  CQ_ERR_TOO_LARGE = 5,     /* the layer does not fit the kernel's shared-memory plan     */
  CQ_ERR_CUDA = 6,          /* a CUDA runtime call failed; see cq_last_cuda_error()       */
  CQ_ERR_NO_DEVICE = 7,     /* no CUDA device, or device is not compute capability 10.x   */
  CQ_ERR_DEVICE_TIMEOUT = 8,/* a bounded device-side wait ran out (reported by cq_poll)   */
  CQ_ERR_UNSUPPORTED = 9,   /* valid request that this build has no kernel for            */
  CQ_ERR_STATIC_LIMIT = 10  /* request exceeds the built-in scratch of cq_layer_matvec_static */
} cq_status;

const char* cq_strerror(int status);
/* cudaError_t of the last failing CUDA call on this thread, 0 if none. */
int cq_last_cuda_error(void);
/* Library ABI version (bumped when a signature changes). */
int cq_abi_version(void);

/* ------------------------------------------------------------------------
 * Prepared layer: the B200 stream layout of one quantized linear.
 * ---------------------------------------------------------------------- */
typedef struct cq_layer {
  /* problem */
  int32_t bits, K, N, C, G;
  /* derived (filled by cq_layer_init) */
  int32_t Kc;          /* K - C, compacted width                                        */
  int32_t Kp;          /* Kc rounded up to 128                                          */
  int32_t Cp;          /* C rounded up to 16                                            */
  int32_t n_gran;      /* 128-column granules per 16-row sub-tile = Kp / 128             */
  int32_t n_sub;       /* 16-row sub-tiles = ceil(N / 16)                               */
  int32_t sets;        /* scale sets per granule: 1 (G % 128 == 0) or 2 (G == 64)        */
  int32_t gran_bytes;  /* bytes of one granule: 16 rows x 128 codes + scales             */
  int32_t cher_bytes;  /* bytes of one sub-tile's cherry block                           */
  /* sections of the device blob */
  uint64_t off_stream, off_cherry, off_osh, off_cidx, blob_bytes;
  void* blob;          /* device memory, blob_bytes long, 256-byte aligned               */
} cq_layer;

/* Fills the derived fields and section offsets for the given problem; no GPU work.
 * blob may be NULL to query blob_bytes. */
int cq_layer_init(cq_layer* layer, int bits, int K, int N, int C, int G, void* blob);

/* GPU re-pack: reference buffers -> stream layout in layer->blob. */
int cq_layer_prepare(const cq_layer* layer, const uint8_t* qweight, const void* scales_f16,
                     const void* cherry_weight_f16, const int16_t* cherry_indices,
                     cq_stream_t stream);

/* Inverse GPU re-pack: stream layout -> reference buffers (byte-identical round trip). */
int cq_layer_unprepare(const cq_layer* layer, uint8_t* qweight, void* scales_f16,
                       void* cherry_weight_f16, int16_t* cherry_indices, cq_stream_t stream);

/* Bytes of scratch the matvec needs on a device (cross-CTA partial sums and flags).
 * The scratch must be zero-filled once before its first use and must not be shared
 * by launches that can overlap on the GPU. */
size_t cq_scratch_bytes(void);

/* y (M, N) fp16 = [y +] x (M, K) fp16 . W^T, M >= 1.  ldx / ldy are row strides in
 * elements.  accumulate != 0 adds to y like the reference's `mul +=`.
 * status_word: device uint32 that receives CQ_ERR_DEVICE_TIMEOUT bits, may be NULL. */
int cq_layer_matvec(const cq_layer* layer, const void* x_f16, int ldx, void* y_f16, int ldy,
                    int M, int accumulate, void* scratch, uint32_t* status_word,
                    cq_stream_t stream);

/* Self-test of the bounded device-side waits (no counterpart in the reference, whose kernels do
 * not wait on one another): a one-warp kernel waits on a barrier that is never completed, gives
 * up after about one second, sets bit 0 of *status_word (device memory) and returns normally. */
int cq_selftest_bounded_wait(uint32_t* status_word, cq_stream_t stream);

/* cq_layer_matvec without a scratch argument and without any allocation (no counterpart in the
 * reference, whose kernels accumulate with atomicAdd and need no scratch,
 * csrc/quant_cuda_kernel.cu:670, :833).  For callers that have no scratch buffer to hand over and may
 * not allocate one: runtimes whose device memory is planned up front, plugins living in another
 * process's memory pool, latency-critical loops where an allocation would stall the device.  The
 * cross-CTA partial sums and flags live in a fixed array inside the library's device image
 * (263,168 bytes per device).
 *   Limits: 1 <= M <= 16 (one launch), a device with at most 256 SMs, and a layer whose M rows fit
 *   one launch's shared-memory plan; otherwise CQ_ERR_STATIC_LIMIT and nothing is launched.
 *   Every call on a device shares the array: calls that can overlap on the GPU (other streams,
 *   other threads) race and must be serialised by the caller.  Each call clears the flags on
 *   `stream` before its launch.
 *   The first call on each device also resolves the array's device address; make that call
 *   before beginning any stream capture on the device.
 * Results are identical to cq_layer_matvec's for the same arguments. */
int cq_layer_matvec_static(const cq_layer* layer, const void* x_f16, int ldx, void* y_f16, int ldy,
                           int M, int accumulate, uint32_t* status_word, cq_stream_t stream);

/* ------------------------------------------------------------------------
 * Row-tile prepared layer: the format of the ONE-activation-row decode matvec (the batch-1 case
 * of csrc/quant_cuda_kernel.cu:718-835 and :558-672, :316-438 of the reference).  Tiles of 16
 * consecutive output rows, one contiguous record per tile, records back to back:
 *   groups  [group of 128 compact columns][256 x bits bytes]: the 16 x 128 codes as A fragments of
 *             mma.sync.m16n8k32 (u8).  Lane 4 g8 + t; register j of a 32-column chunk = row
 *             g8 + 8 (j & 1), columns 16 (j >> 1) + 4 t + b in byte b.
 *             4-bit: [load l = 0, 1][lane][16 B]; word j = register j of chunk 2 l (low nibbles)
 *                    and of chunk 2 l + 1 (high nibbles).
 *             3-bit: per 64-column half s words A, B, C: [lane][16 B] = A0 B0 C0 A1, then
 *                    [lane][8 B] = B1 C1.  Word wi: register wi of chunk 2 s in bits 0-2 and of chunk
 *                    2 s + 1 in bits 4-6 of its bytes; register 3 as bit planes: code bit wi of chunk
 *                    2 s (2 s + 1) in bit 3 (bit 7) of word wi.
 *   scales  [group][set][g8][row g8, row g8 + 8] fp16 (set = 64-column half, only for 64-wide groups)
 *   cherry  [block of 16 cherry columns][lane][16 B]: A fragments of mma.sync.m16n8k16 (fp16)
 * followed by
 *   perm    [groups x 128] uint16: original column of each compact column, K past K'
 *   cidx    [Cp] uint16 sorted cherry columns, K past C
 *   work    only for layers of more than 64 groups (K - C > 8192), whose tiles are shared by ksplit
 *           CTAs, each taking a part of the columns: [ksplit][NT][4][16] fp32 partial sums and [NT]
 *           uint32 arrival counters (zeroed by cq_rlayer_prepare, left zero by every launch).  The
 *           CTA that arrives last adds the parts in part order, so results do not depend on timing.
 *           Launches of such a layer that can overlap on the GPU (different streams) would share
 *           this area: serialise them.
 * Same role as cq_layer; no caller-provided scratch.
 * ---------------------------------------------------------------------- */
typedef struct cq_rlayer {
  int32_t bits, K, N, C, G;
  int32_t Kc;          /* K - C                                                          */
  int32_t NG;          /* 128-column groups per row = ceil(Kc / 128)                     */
  int32_t sets;        /* scale sets per group: 1 (G % 128 == 0) or 2 (G == 64)          */
  int32_t Cp;          /* C rounded up to 16                                             */
  int32_t NT;          /* 16-row tiles = ceil(N / 16)                                    */
  int32_t tile_bytes;  /* NG * 256 * bits + NG * sets * 32 + Cp / 16 * 512               */
  int32_t ksplit;      /* CTAs that share a tile, each taking NG / ksplit groups: ceil(NG / 64) */
  uint64_t off_tiles, off_perm, off_cidx, off_work, blob_bytes;
  void* blob;          /* device memory, blob_bytes long, 256-byte aligned               */
} cq_rlayer;

int cq_rlayer_init(cq_rlayer* layer, int bits, int K, int N, int C, int G, void* blob);
int cq_rlayer_prepare(const cq_rlayer* layer, const uint8_t* qweight, const void* scales_f16,
                      const void* cherry_weight_f16, const int16_t* cherry_indices,
                      cq_stream_t stream);
/* Inverse re-pack (byte-identical round trip). */
int cq_rlayer_unprepare(const cq_rlayer* layer, uint8_t* qweight, void* scales_f16,
                        void* cherry_weight_f16, int16_t* cherry_indices, cq_stream_t stream);
/* CQ_OK if cq_rlayer_matvec can run this layer on the current device, else the status it would
 * return (CQ_ERR_UNSUPPORTED / CQ_ERR_TOO_LARGE); no GPU work. */
int cq_rlayer_check(const cq_rlayer* layer);
/* y (N) fp16 = [y +] x (K) fp16 . W^T, one activation row; allocates nothing, needs no scratch.
 * CQ_ERR_UNSUPPORTED for layers outside the kernel's envelope (more than 256 cherry columns, or more
 * than 248 cherry columns inside one warp's column range) and
 * CQ_ERR_TOO_LARGE when not even two tiles fit shared memory: use cq_layer_matvec for those.
 * status_word: device uint32 that receives CQ_ERR_DEVICE_TIMEOUT bits if a bounded wait on the
 * kernel's own bulk copies ever runs out; may be NULL. */
int cq_rlayer_matvec(const cq_rlayer* layer, const void* x_f16, void* y_f16, int accumulate,
                     uint32_t* status_word, cq_stream_t stream);
/* The down projection of a gated MLP with the SwiGLU folded into its input staging:
 *   y (M, N) fp16 = (silu(gate) * up) (M, K) . W^T
 * (the reference's LlamaMLP.forward, llama/modeling_llama_quant.py, computes act_fn(gate_proj(x)) *
 * up_proj(x) as separate PyTorch ops before down_proj).  The product is formed with the roundings of
 * those ops (the activation is rounded to fp16, then an fp16 multiplication), so the result equals
 * cq_rlayers_matvec on the separately computed product bit for bit.  gate and up share the row stride. */
int cq_rlayer_matvec_swiglu(const cq_rlayer* layer, const void* gate_f16, const void* up_f16, int ld,
                            void* y_f16, int ldy, int M, uint32_t* status_word, cq_stream_t stream);
/* The largest batch for which cq_rlayers_matvec is the faster path for this layer (beyond it
 * cq_tlayer_gemm is): 12 for layers of up to 8192 quantized columns, 8 for wider ones, 0 for layers
 * the kernel does not take.  No GPU work. */
int cq_rlayer_preferred_rows(const cq_rlayer* layer);
/* cq_rlayer_matvec for callers that hold their activations in HOST memory (a foreign-function
 * binding with no device tensors of its own; the reference's op only takes device tensors,
 * csrc/quant_cuda.cpp:56-69): copies x_host (K fp16) to the device staging buffer x_dev, runs the
 * kernel into y_dev, copies the N fp16 results to y_host and returns when y_host is complete (the
 * stream is synchronised).  With page-locked (mapped) host buffers no copy engine is involved: a
 * one-CTA kernel fetches x across the bus while the matvec already streams its weights, and the
 * matvec stores y straight into y_host.  Pageable memory works (two asynchronous copies).
 * x_dev / y_dev: device memory of K and N fp16 owned by the caller, x_dev 16-byte aligned. */
int cq_rlayer_matvec_host(const cq_rlayer* layer, const void* x_host_f16, void* y_host_f16,
                          void* x_dev_f16, void* y_dev_f16, uint32_t* status_word,
                          cq_stream_t stream);
/* The general form: up to 4 layers that take the same activations (q / k / v, gate / up of the
 * reference's LLaMA, llama/modeling_llama_quant.py: LlamaAttention.forward, LlamaMLP.forward, which
 * calls them one after the other) in one launch, M >= 1 activation rows:
 *   ys[i] (M, N_i) fp16 = [ys[i] +] x (M, K) fp16 . W_i^T,  ldx / ldy row strides in elements
 * (ldy is shared by the outputs).  The layers must agree in bits, K, cherry count and group size
 * (CQ_ERR_BAD_SHAPE otherwise); the SMs are divided among them in proportion to their rows.  Up to
 * four activation rows ride in one launch (they fill the unused columns of the same integer MMAs:
 * a row more costs about a quarter of a launch); more rows are walked in slices of four, each reading
 * the weights again.
 * Every output element is computed exactly as by cq_rlayer_matvec on that layer and row alone
 * (bit-identical).  Same limits and status word. */
int cq_rlayers_matvec(const cq_rlayer* const* layers, int n_layers, const void* x_f16, int ldx,
                      void* const* ys_f16, int ldy, int M, int accumulate,
                      uint32_t* status_word, cq_stream_t stream);

/* ------------------------------------------------------------------------
 * Element-wise kernels of the decode harness around the quantized linear (fp16 in / out, fp32
 * arithmetic).  In the reference they are PyTorch ops of its vendored LLaMA
 * (llama/modeling_llama_quant.py: LlamaRMSNorm, apply_rotary_pos_emb, LlamaMLP.forward).
 * ---------------------------------------------------------------------- */
/* h = x (+ residual); y = h * rsqrt(mean(h^2) + eps) * weight; h is stored to h_out when not NULL. */
int cq_rmsnorm(const void* x_f16, const void* residual_f16, const void* weight_f16, void* y_f16,
               void* h_out_f16, int rows, int hidden, float eps, cq_stream_t stream);
/* Rotary embedding ("rotate half" convention) of q (T, H, D) and k (T, KV, D) in place at
 * positions[t] (device int64), tables (max_seq, D/2) fp32; k and v rows are written to the caches
 * (sequences, max_seq, KV, D) at the same positions: token t belongs to sequence
 * t / tokens_per_seq (a prompt of T tokens: tokens_per_seq = T; a decode step of B sequences:
 * T = B, tokens_per_seq = 1).  A token whose position is outside [0, max_seq) is left alone:
 * nothing is read from the tables or written to the caches for it. */
int cq_rope_cache(void* q_f16, void* k_f16, const void* v_f16, const float* cos_table,
                  const float* sin_table, const long long* positions, void* k_cache_f16,
                  void* v_cache_f16, int T, int n_heads, int n_kv_heads, int head_dim, int max_seq,
                  int tokens_per_seq, cq_stream_t stream);
/* Single-query attention over the caches (sequences, max_seq, KV, D), one query per sequence:
 * out (sequences, H, D) = softmax(q . K^T * scale) . V over positions
 * 0..min(position[sequence], max_seq - 1) (device int64), grouped-query heads allowed; head_dim
 * divides 256 (the reference calls PyTorch's attention, llama/modeling_llama_quant.py:371-419).
 * The positions of a head are divided among several CTAs so that a decode step fills the GPU; they
 * meet in `workspace`: device memory of cq_attn_decode_workspace_bytes(...) bytes, 16-byte aligned,
 * zero-filled once before its first use (every launch leaves it ready for the next), not shared by
 * launches that can overlap on the GPU. */
size_t cq_attn_decode_workspace_bytes(int sequences, int n_heads, int head_dim, int max_seq);
int cq_attn_decode(const void* q_f16, const void* k_cache_f16, const void* v_cache_f16,
                   const long long* position, void* out_f16, int sequences, int n_heads,
                   int n_kv_heads, int head_dim, int max_seq, float scale, void* workspace,
                   cq_stream_t stream);
/* out = silu(gate) * up, n elements. */
int cq_silu_mul(const void* gate_f16, const void* up_f16, void* out_f16, long long n,
                cq_stream_t stream);

/* ------------------------------------------------------------------------
 * Tile-layout prepared layer: the format of the tcgen05 (UMMA + tensor memory) kernels.
 * 128-row tiles; a granule is 128 rows x 128 compact columns; cherry columns travel in the same
 * stream as fp16 items of 16 columns.  Same role as cq_layer above, different kernel family.
 * ---------------------------------------------------------------------- */
typedef struct cq_tlayer {
  int32_t bits, K, N, C, G;
  int32_t Kc, Kp, Cp;
  int32_t n_gran;      /* granules per row tile = Kp / 128                               */
  int32_t n_tile;      /* row tiles = ceil(N / 128)                                      */
  int32_t n_cher;      /* cherry items per row tile = Cp / 16                            */
  int32_t sets;        /* scale sets per granule: 1 (G % 128 == 0) or 2 (G == 64)        */
  int32_t gran_bytes;  /* 2048 * bits + 256 * sets                                       */
  int32_t tile_bytes;  /* n_cher * 4096 + n_gran * gran_bytes                            */
  uint64_t off_stream, off_cidx, off_osh, blob_bytes;
  void* blob;          /* device memory, blob_bytes long, 256-byte aligned               */
} cq_tlayer;

int cq_tlayer_init(cq_tlayer* layer, int bits, int K, int N, int C, int G, void* blob);
int cq_tlayer_prepare(const cq_tlayer* layer, const uint8_t* qweight, const void* scales_f16,
                      const void* cherry_weight_f16, const int16_t* cherry_indices,
                      cq_stream_t stream);
int cq_tlayer_unprepare(const cq_tlayer* layer, uint8_t* qweight, void* scales_f16,
                        void* cherry_weight_f16, int16_t* cherry_indices, cq_stream_t stream);
/* Prefill GEMM: y (M, N) fp16 = [y +] x (M, K) fp16 . W^T for many activation rows, on the tcgen05
 * tensor cores (weights dequantised to fp16 on the fly into tensor memory, fp32 accumulation).
 * Replaces the reference's dense mode, QuantLinear.unpack() followed by F.linear
 * (llama/qlinear.py:183-195), and its batched kernels for large batches
 * (csrc/quant_cuda_kernel.cu:718-835).  `workspace` is device memory of at least
 * cq_tlayer_gemm_workspace_bytes(layer, M) bytes, 128-byte aligned, for the staged activations;
 * launches that can overlap on the GPU need separate workspaces. */
size_t cq_tlayer_gemm_workspace_bytes(const cq_tlayer* layer, int M);
int cq_tlayer_gemm(const cq_tlayer* layer, const void* x_f16, int ldx, void* y_f16, int ldy, int M,
                   int accumulate, void* workspace, uint32_t* status_word, cq_stream_t stream);

/* ------------------------------------------------------------------------
 * Drop-in operator entry points (reference: csrc/quant_cuda.cpp:41-69, 26-38).
 * Dimension arguments are what the reference derives from its tensors
 * (csrc/quant_cuda_kernel.cu:686-690):
 *   height = qweight.size(0), width = N = qweight.size(1), batch = vec.size(0),
 *   vec_height = K = vec.size(1), cherry_size = C.
 * `mul` is accumulated into (the caller pre-zeroes it, llama/qlinear.py:177).
 * The re-packed layer is cached inside the library, keyed by the four buffer
 * addresses, the dimensions and version_tag (pass any value that changes when
 * the buffers' contents change, e.g. a sum of tensor version counters); a copy
 * is made per kernel family actually used (1 row / 2..7 rows / 8 rows and more).
 * Addresses alone do not identify a buffer for ever: call cq_cache_evict when the
 * buffers are freed or re-filled.
 * ---------------------------------------------------------------------- */
int cq_vecquant4matmul_cherryq(const void* vec_f16, const uint8_t* qweight,
                               const void* cherry_weight_f16, const int16_t* cherry_indices,
                               const void* scaling_factors_f16, void* mul_f16,
                               int batch, int vec_height, int height, int width,
                               int cherry_size, int group_size, uint64_t version_tag,
                               cq_stream_t stream);

/* fp16 != 0: half x / scales / cherry / mul and int16 indices.
 * fp16 == 0: float x / scales / cherry / mul and int32 indices
 * (csrc/quant_cuda_kernel.cu:139-179). */
int cq_vecquant3matmul_cherryq(const void* vec, const uint8_t* qweight,
                               const void* cherry_weight, const void* cherry_indices,
                               const void* scaling_factors, void* mul,
                               int batch, int vec_height, int height, int width,
                               int cherry_size, int group_size, int fp16,
                               uint64_t version_tag, cq_stream_t stream);

/* out[k', n] = (u - (2^(bits-1) - 0.5)) * scaling_factors[k' / group_size, n], fp32,
 * for the K' = height - cherry_size compacted columns
 * (csrc/quant_cuda_kernel.cu:838-922 and 925-1010; the 4-bit version implements what
 * the reference intends, not its block-height slip at :934/:964). */
int cq_dequantize3_normal(const uint8_t* qweight, const float* scaling_factors, float* out,
                          int qrows, int width, int height, int cherry_size, int group_size,
                          cq_stream_t stream);
int cq_dequantize4_normal(const uint8_t* qweight, const float* scaling_factors, float* out,
                          int qrows, int width, int height, int cherry_size, int group_size,
                          cq_stream_t stream);

/* Drop every cached re-packed layer (frees device memory). */
int cq_cache_clear(void);
/* Drop the cached copies made from this set of buffer addresses on the current device (the
 * reference's ops keep no references, csrc/quant_cuda.cpp:56-69: a caller that frees or re-uses
 * the buffers tells the cache so; the torch module does it by watching the tensors' storages). */
int cq_cache_evict(const void* qweight, const void* scales_f16, const void* cherry_weight_f16,
                   const void* cherry_indices);
/* Number of cached layers and the bytes they hold. */
int cq_cache_stats(int* n_layers, uint64_t* bytes);

/* Reads and clears the library's per-device status word (host call, synchronises
 * the given stream).  Returns CQ_OK or CQ_ERR_DEVICE_TIMEOUT. */
int cq_poll(cq_stream_t stream);

/* ------------------------------------------------------------------------
 * Packing (reference: llama/qlinear.py:67-118) and dense unpacking (:120-162).
 * ---------------------------------------------------------------------- */
/* weight: (N, K) row-major, fp16 (weight_is_f32 == 0) or fp32.
 * cherry_unsorted: int32 (C,) distinct column indices in any order.
 * Outputs in the reference formats above.  tmp: device scratch of
 * cq_pack_tmp_bytes(K) bytes. */
size_t cq_pack_tmp_bytes(int K);
int cq_pack(const void* weight, int weight_is_f32, const int32_t* cherry_unsorted,
            int bits, int K, int N, int C, int G,
            uint8_t* qweight, void* scales_f16, void* cherry_weight_f16,
            int16_t* cherry_indices, void* tmp, cq_stream_t stream);

/* dense: (N, K) fp16 = what QuantLinear.unpack() returns. */
int cq_unpack_dense(const uint8_t* qweight, const void* scales_f16,
                    const void* cherry_weight_f16, const int16_t* cherry_indices,
                    int bits, int K, int N, int C, int G, void* dense_f16,
                    cq_stream_t stream);

/* ------------------------------------------------------------------------
 * Exchange step of the column-parallel layer over peer memory (no counterpart in the reference,
 * which runs on one GPU: its llama/qlinear.py:164-199 forward produces the whole output vector).
 * Every rank holds N / P output columns; one small kernel per rank stores its (rows, cols_local)
 * fp16 slice into a landing area of every rank with plain peer stores, each 8-byte word carrying
 * 4 payload bytes and the call's sequence number, polls its own landing area until every word
 * carries that number (bounded by timeout_ms, then CQ_ERR_DEVICE_TIMEOUT bits in *status_word and
 * the output is filled with NaN) and writes the gathered (rows, P * cols_local) fp16 matrix.
 * One rank per GPU: ranks never share a device.  Every rank makes the same sequence of calls.
 *
 * A region is cq_peer_region_bytes(capacity) bytes of device memory, zeroed at creation (its header
 * keeps the capacity: a call that states another one sends nothing and reports like a time-out);
 * capacity (a multiple of 16) bounds 4 * rows * cols_local * P of one call (twice the payload).
 * Peers map it through the 64-byte CUDA IPC handle.  regions[] holds P device pointers,
 * regions[rank] the own one.
 * Creation, export, open, close and destroy are host calls that synchronise; the gather itself
 * is one launch on the given stream and can be captured.
 * ---------------------------------------------------------------------- */
#define CQ_PEER_MAX_RANKS 8
size_t cq_peer_region_bytes(size_t capacity);
int cq_peer_region_create(size_t capacity, void** region);
int cq_peer_region_destroy(void* region);
int cq_peer_region_export(const void* region, unsigned char handle[64]);
int cq_peer_region_open(const unsigned char handle[64], void** region);
int cq_peer_region_close(void* region);
int cq_peer_allgather(void* const* regions, int world, int rank, size_t capacity, const void* x_f16,
                      void* out_f16, int rows, int cols_local, int timeout_ms,
                      uint32_t* status_word, cq_stream_t stream);
/* cq_rlayers_matvec on one layer shard followed by the exchange in the SAME launch: every CTA stores
 * its rows of the local slice y_local (M, N) fp16 (contiguous, 8-byte aligned, 1 <= M <= 4), the CTA
 * of the grid that finishes last runs the exchange described above (same regions, same call sequence
 * as cq_peer_allgather: the two may be mixed, every rank making the same sequence of calls) and
 * y_all (M, P * N) fp16 is complete when the next kernel of the stream starts.  Saves the kernel
 * boundary between the matvec and the exchange. */
int cq_rlayer_matvec_gather(const cq_rlayer* layer, const void* x_f16, int ldx, void* y_local_f16,
                            int M, void* const* regions, int world, int rank, size_t capacity,
                            void* y_all_f16, int timeout_ms, uint32_t* status_word,
                            cq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CHERRYQ_H_ */
