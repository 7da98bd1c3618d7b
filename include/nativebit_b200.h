/* nativebit_b200 — C ABI of the B200 (sm_100a) packed-inference kernels.
 *
 * This is the boundary a NativeBit maintainer binds instead of the reference's JIT-built
 * kernels.  Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (cudaStream_t passed as void*; NULL = the legacy default stream), launches asynchronously on
 * that stream, never allocates or frees device memory, never synchronises, and returns an
 * nb_status (0 = ok).  There is no CPU fallback: on a machine without a usable sm_100 device
 * the compute entry points return NB_ERR_ARCH or NB_ERR_LAUNCH.
 *
 * Packed layout: exactly the bytes nativebit/pack.py writes (pack_3bit :21-41, pack_nbits
 * :97-116, pack_4bit :75-82), weights flat in row-major (out_features, in_features) order, one
 * codebook of 2^bits entries per `block_size` consecutive weights.
 */
#ifndef NATIVEBIT_B200_H_
#define NATIVEBIT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  NB_OK = 0,
  NB_ERR_ARG = 1,       /* null pointer, bad enum, non-positive size */
  NB_ERR_ALIGN = 2,     /* a pointer is not aligned as the kernel needs (16 bytes) */
  NB_ERR_SHAPE = 3,     /* shape not supported by the fast kernels (see each function) */
  NB_ERR_ARCH = 4,      /* current device is not compute capability 10.x */
  NB_ERR_LAUNCH = 5,    /* the CUDA runtime refused the launch; see nb_last_cuda_error() */
  NB_ERR_TIMEOUT = 6,   /* a bounded device-side wait ran out (tensor-parallel paths only) */
  NB_ERR_WORKSPACE = 7  /* workspace missing or smaller than nb_*_workspace_bytes() */
} nb_status;

typedef enum { NB_F32 = 0, NB_F16 = 1, NB_BF16 = 2 } nb_dtype;

/* Library version (major*10000 + minor*100 + patch) and a printable name for a status. */
int nb_version(void);
const char* nb_status_string(int status);
/* Text of the last CUDA runtime error seen by this thread inside the library ("" if none). */
const char* nb_last_cuda_error(void);

/* CPU-only self check of the in-register unpack tables (no GPU needed): returns NB_OK when the
 * selector scheme used by the kernels reproduces every index position for random packed
 * blocks at 2 and 3 bits.  No counterpart in the reference; used by the CPU test-suite. */
int nb_selftest_tables(void);

/* ---- bit-unpack:  replaces nativebit/pack.py:44-68 (unpack_3bit), :85-90 (unpack_4bit),
 * :119-138 (unpack_nbits, bits=2) and the per-forward unpack of
 * inference/triton_kernel.py:262-269 / inference/generate_torch.py:165-173.
 * packed: ceil(count*bits/8) bytes for bits 2/4, 3*ceil(count/8) bytes for bits 3 (device).
 * idx_out: count bytes (device), one index per byte.  bits in {2,3,4}. */
int nb_unpack(const uint8_t* packed, int bits, int64_t count, uint8_t* idx_out, void* stream);

/* ---- bit-pack on device: replaces inference/triton_kernel.py:199-220 (pack_indices_to_3bit)
 * and nativebit/pack.py:21-41 / :75-82 / :97-116 for bits in {2,3,4}.  `packed_out` must hold
 * the byte counts given for nb_unpack; padding indices are zero as in the reference. */
int nb_pack(const uint8_t* idx, int bits, int64_t count, uint8_t* packed_out, void* stream);

/* ---- dequantise a whole weight: replaces nativebit/pack.py:145-169 (reconstruct_weight) and the
 * gather of nativebit/inference.py:44-45.  W[r][c] = codebook[b][idx[b][t]] with
 * b*block_size+t = r*n_cols+c; bit-exact (the values are the codebook entries converted to
 * w_dtype; fp16 -> fp32 and fp16 -> fp16 are exact, -> bf16 rounds to nearest even).
 * codebook: (ceil(n_rows*n_cols/block_size), 2^bits) of cb_dtype (NB_F16 or NB_F32).
 * Any block_size >= 1 and bits in {2,3,4}; total weights need not fill the last block. */
int nb_dequant(const uint8_t* packed, const void* codebook, int cb_dtype, int bits, int block_size,
               int64_t n_rows, int64_t n_cols, void* w_out, int w_dtype, void* stream);

/* ---- quantise a dense weight against its codebooks on the device: replaces the exporter's
 * argmin, nativebit/pack.py:176-199 (_compute_indices, L1 distance, no active mask) and
 * inference/pack.py:21-35 (quantize_weight, squared distance: the same argmin).
 * idx_out[i] = argmin_e |w[i] - codebook[i/block_size][e]| (first minimum on ties) for
 * i < ceil(total/block_size)*block_size; weights past `total` count as 0.  w: fp32 device array of
 * `total` values in row-major weight order; n_entries 2..256. */
int nb_quantize(const float* w, int64_t total, const void* codebook, int cb_dtype, int n_entries, int block_size,
                uint8_t* idx_out, void* stream);

/* ---- fused decode GEMV / skinny GEMM (M = 1..16 activation rows):
 * y[m][n] = sum_k W[n][k] * x[m][k].  Replaces inference/cuda_kernel.py:38-104
 * (dequant_matvec_3bit_kernel + wrapper), inference/triton_kernel.py:144-196 (Triton 3-bit kernel)
 * and, for 2 <= M <= 16, the unpack+gather+matmul of inference/triton_kernel.py:258-275.
 * x: (M, K) row-major of x_dtype; y: (M, N) row-major of y_dtype; fp32 accumulation.
 * bits in {2,3,4} (codebooks of 4, 8, 16 entries; 4-bit in the nativebit/pack.py:75-90 nibble layout);
 * block_size 128; K % 128 == 0.
 * packed and codebook must be 16-byte aligned.  Weights enter the tensor-core contraction as
 * exact fp16 values (an fp32 codebook is rounded to fp16).  bf16/fp16 activations enter as fp16
 * (exact for bf16 inputs of magnitude 6.1e-5..65504; larger magnitudes are clamped); fp32
 * activations enter as the sum of two fp16 terms (about 22 significant bits).
 * workspace: device scratch of at least nb_gemv_workspace_bytes() bytes whose first 16 KB were
 * zero-filled once before its first use; it is then owned by calls on one stream at a time.
 * The first 16 KB hold ticket counters, which every launch leaves zeroed, and a status word
 * (int index 4095) that a launch sets to NB_ERR_TIMEOUT if a bounded wait ran out; the rest
 * carries the partial sums of split-K launches.  One workspace may serve launches of
 * different shapes.  Weights and codebooks are requested before the kernel waits for earlier
 * work of the stream (programmatic dependent launch), so they must not be written by any kernel or
 * copy of the stream that may still be in flight (use nb_gemv_ordered then); x and y are touched
 * only after that wait. */
size_t nb_gemv_workspace_bytes(int M, int N, int K, int bits, int block_size);
int nb_gemv(const void* x, int x_dtype, int M, const uint8_t* packed, const void* codebook, int cb_dtype,
            int bits, int block_size, int N, int K, void* y, int y_dtype, void* workspace,
            size_t workspace_bytes, void* stream);
/* nb_gemv launched fully stream-ordered (no early start): use it when `packed` or `codebook` were
 * written by ANY earlier kernel or copy of the same stream that may still be in flight (e.g. nb_pack
 * directly before it, as in inference/triton_kernel.py:119-140 where the indices are packed per call).
 * nb_gemv itself requests its weights before it waits for earlier work of the stream. */
int nb_gemv_ordered(const void* x, int x_dtype, int M, const uint8_t* packed, const void* codebook, int cb_dtype,
                    int bits, int block_size, int N, int K, void* y, int y_dtype, void* workspace,
                    size_t workspace_bytes, void* stream);

/* ---- prefill GEMM (many activation rows) on the tcgen05 tensor cores:
 * y (M, N) = x (M, K) . W^T.  Replaces the unpack + gather + matmul of
 * inference/triton_kernel.py:258-275 for large M and follows the any-M contract of
 * nativebit_jax/packed_kernel.py:86-97, 151-178 (16-bit operands, fp32 accumulation) with one
 * difference: the weights enter as the fp16 codebook entries themselves (exact), not rounded to bf16,
 * and the bf16 activations are converted to fp16 (exact for magnitudes 6.1e-5..65504, clamped above).
 * x: (M, K) NB_BF16, NB_F16 or NB_F32 (two fp16 terms per element in adjacent operand rows, their results added
 * in the epilogue) row-major, 16-byte aligned; y: (M, N) NB_BF16 or NB_F32; K % 64 == 0 and
 * K % block_size == 0; bits in {2,3,4}.  `workspace` must be 256-byte aligned and hold
 * nb_prefill_workspace_bytes(M, N, K) bytes: its first 256 bytes carry a status word that must be
 * zero before the first call and is set to NB_ERR_TIMEOUT if a bounded wait inside the kernel ran
 * out; the rest is scratch (dequantised weights, fp16 activations). */
size_t nb_prefill_workspace_bytes(int M, int N, int K);
int nb_gemm_prefill(const void* x, int x_dtype, int M, const uint8_t* packed, const void* codebook, int cb_dtype, int bits,
                    int block_size, int N, int K, void* y, int y_dtype, void* workspace, size_t workspace_bytes,
                    void* stream);

/* ---- prefill GEMM with the dequantisation fused into the tensor-core kernel: producer warps turn the
 * packed weights into fp16 tiles in shared memory, tcgen05.mma consumes them; no dense copy of W is ever
 * written to global memory.  Same contract as nb_gemm_prefill (the reference's M > 1 path,
 * inference/triton_kernel.py:258-275; tile-wise dequantise-and-contract as in
 * nativebit_jax/packed_kernel.py:135-178; exact fp16 weights, fp32 accumulation) for any M >= 1, but the
 * weights are given in the stream layout (nb_stream_pack with row_mode 0) instead of the pack.py bytes.
 * x: (M, K) NB_F16, NB_BF16 (converted to fp16 into the workspace first) or NB_F32 (carried as two fp16 terms per
 * element, hi = fp16(x) and lo = fp16(x - hi), as two operand rows whose results the kernel adds: about 22
 * significant bits, as in nb_gemv), 16-byte aligned;
 * K % 128 == 0; y: (M, N) NB_BF16 or NB_F32.  workspace: nb_prefill_fused_workspace_bytes(M, N, K) bytes,
 * 256-byte aligned; its first 256 bytes carry a status word (zero before the first call; NB_ERR_TIMEOUT
 * if a bounded wait inside the kernel ran out), then the fp16 copy of the activations and, for short
 * inputs, fp32 slabs: when the output has fewer 128 x BN tiles than half the SMs, the k range is cut
 * into up to 8 parts that run on different SMs and a second kernel adds their results in k order (still
 * bit-identical from run to run). */
size_t nb_prefill_fused_workspace_bytes(int M, int N, int K);
int nb_gemm_prefill_fused(const void* x, int x_dtype, int M, const uint8_t* w_stream, int bits, int N, int K, void* y,
                          int y_dtype, void* workspace, size_t workspace_bytes, void* stream);

/* The tensor-core kernel alone: y (M, N) = x (M, K) . w (N, K)^T with x and w bf16 row-major
 * (16-byte aligned, K % 64 == 0), y NB_BF16 or NB_F32, fp32 accumulation in tensor memory.
 * `status` is a device int (zero before the first call) or NULL.  No counterpart in the
 * reference, which calls a library matmul here. */
int nb_gemm_bf16(const void* x, const void* w, int M, int N, int K, void* y, int y_dtype, int* status, void* stream);

/* ---- decode-step glue (one new token per sequence, fp32 activations, position read from device
 * memory so the step replays from a CUDA graph).  They restate the reference's cached decode path,
 * inference/generate_torch.py: RMSNorm :29-38, RoPE on interleaved pairs :41-60, cache write and
 * attention over the valid prefix :86-97, SwiGLU :116-117.
 * nb_add_rmsnorm: x (B, C) += delta (may be NULL); out = x / sqrt(mean(x^2) + eps) * w; C <= 4096.
 * nb_rope_kv_write: qkv (B, 3*H*hd) = [q|k|v] of this rank's H heads; cos2/sin2 (ctx, hd) are the
 *   per-pair tables repeated twice; rotated k and v go to the caches (B, H, ctx, hd) at *pos, rotated
 *   q to q_out (B, H, hd).
 * nb_decode_attention: softmax(q . K[0..*pos] / sqrt(hd)) . V[0..*pos] per head, written to
 *   out[b*out_stride + out_offset + h*hd + d]; hd a multiple of 4, <= 128; caches 16-byte aligned.  The
 *   keys of a head are split over a cluster of up to 8 CTAs, merged through distributed shared memory.
 *   Launched with programmatic stream serialization, the attention kernels read *pos, the rotary entries and the
 *   cache rows below *pos BEFORE their dependency wait: these must have been written at least two launches earlier
 *   (a decode loop writes them in the step before), and the launch directly before must not release its dependents
 *   ahead of its own dependency wait (the matvec, norm, rope and glue kernels of this library release after it; a
 *   launch without the attribute never releases early).
 * nb_silu_mul: hmid (B, F) = silu(gu[:, :F]) * gu[:, F:]. */
int nb_add_rmsnorm(float* x, const float* delta, const float* w, float eps, float* out, int B, int C, void* stream);
int nb_rope_kv_write(const float* qkv, int B, int H, int hd, const float* cos2, const float* sin2, const int64_t* pos,
                     float* k_cache, float* v_cache, int ctx, float* q_out, void* stream);
int nb_decode_attention(const float* q, const float* k_cache, const float* v_cache, const int64_t* pos, int B, int H,
                        int hd, int ctx, float* out, int out_stride, int out_offset, void* stream);
int nb_silu_mul(const float* gu, int B, int F, float* hmid, void* stream);
/* Causal attention of a prompt of T tokens per sequence that continues a cache of pos0 keys (pos0 = 0 for a fresh
 * prompt), one launch per layer: rotates q and k of qkv (B*T, 3*H*hd) with rows pos0 .. pos0+T-1 of cos2/sin2, writes
 * the rotated k and v to the caches (B, H, ctx, hd) at those positions and
 * out[(b*T + t)*out_stride + out_offset + h*hd + d] = softmax(q_t . K[0..pos0+t] / sqrt(hd)) . V[0..pos0+t]
 * (inference/generate_torch.py:41-60, :86-97 for T > 1).  fp32 throughout; hd a multiple of 4, <= 128; pos0 + T <= ctx;
 * qkv, caches and out 16-byte aligned, out_stride and out_offset multiples of 4. */
int nb_prefill_attention(const float* qkv, int B, int T, int H, int hd, const float* cos2, const float* sin2, int pos0,
                         float* k_cache, float* v_cache, int ctx, float* out, int out_stride, int out_offset, void* stream);
/* nb_rope_kv_write and nb_decode_attention in one launch: rotates q and k of qkv (B, 3*H*hd), writes
 * k and v to the caches at *pos and attends with the rotated q (same limits as nb_decode_attention). */
int nb_decode_attention_rope(const float* qkv, const float* cos2, const float* sin2, const int64_t* pos, float* k_cache,
                             float* v_cache, int B, int H, int hd, int ctx, float* out, int out_stride, int out_offset,
                             void* stream);

/* The two ends of a decode step (inference/generate_torch.py:142-160: embedding lookup; tied LM head,
 * 30*tanh(x/30) soft-cap; :300-310 greedy argmax), for one sequence per CTA.
 * nb_embed_rows: out (B, C) fp32 = table[token[b], :] of a bf16 (V, C) table.
 * nb_softcap_argmax: logits (B, V) NB_BF16 or NB_F32 -> logits_out (B, V) fp32 = cap * tanh(x / cap);
 *   token[b] = index of the largest capped logit (lowest index among equals); *pos += 1 if pos != NULL. */
int nb_embed_rows(const void* table_bf16, const int64_t* token, int B, int V, int C, float* out, void* stream);
int nb_softcap_argmax(const void* logits, int logits_dtype, int B, int V, float cap, float* logits_out, int64_t* token,
                      int64_t* pos, void* stream);
/* The tied LM head of ONE sequence with both ends of it in the same two launches (inference/generate_torch.py:155-160,
 * :300-310): logits_out (V) fp32 = cap * tanh(dot(table[v], h) / cap) with h = rmsnorm(x + delta) * norm_weight (delta may
 * be NULL; norm_weight NULL: h = x + delta), token[0] = index of the largest capped logit (lowest index among equals),
 * *pos += 1 if pos != NULL.  table: bf16 (V, C), C a multiple of 256 up to 3072; products are exact in fp32.  scratch:
 * nb_lm_head_scratch_bytes() bytes, 16-byte aligned (per-CTA arg-max candidates). */
size_t nb_lm_head_scratch_bytes(void);
int nb_lm_head(const float* x, const float* delta, const float* norm_weight, float eps, const void* table_bf16, int V, int C,
               float cap, float* logits_out, int64_t* token, int64_t* pos, void* scratch, void* stream);

/* ---- nb_gemv with the preceding element-wise step of the decoder folded into the staging of its
 * activations, so the step needs no separate launch for it (fp32 activations, M <= 8; everything
 * else as nb_gemv).  The reference runs these as separate torch ops around each packed linear
 * (inference/generate_torch.py:29-38 RMSNorm, :109-117 residual adds and SwiGLU).
 *  NB_PRO_ADD_RMSNORM: v = x (M, K) + delta (M, K, may be NULL);
 *      activation = v / sqrt(mean(v^2) + eps) * norm_weight (K);  v is also written to x_out (M, K; may
 *      be NULL; must not be x: other CTAs still read x).  Equal to nb_add_rmsnorm followed by nb_gemv up
 *      to rounding: the factor 1/rms, a scalar per row, is applied to the output instead of the activations.
 *  NB_PRO_SILU_MUL: x is (M, 2K) = [gate | up]; activation = silu(gate) * up, as nb_silu_mul;
 *      delta, norm_weight, x_out, eps are ignored.
 * x, delta, norm_weight, x_out 16-byte aligned. */
typedef enum { NB_PRO_NONE = 0, NB_PRO_ADD_RMSNORM = 1, NB_PRO_SILU_MUL = 2 } nb_prologue;
int nb_gemv_fused(int prologue, const float* x, const float* delta, const float* norm_weight, float eps, float* x_out,
                  int M, const uint8_t* packed, const void* codebook, int cb_dtype, int bits, int block_size, int N,
                  int K, void* y, int y_dtype, void* workspace, size_t workspace_bytes, void* stream);

/* ---- tensor-parallel decode: the all-reduce after a row-sharded projection folded into the GEMVs on
 * both sides of it, so that no collective kernel runs between them (the reference has no multi-GPU
 * inference; the library equivalent is nb_gemv, an NCCL all_reduce, nb_add_rmsnorm, nb_gemv).
 *  push   = 1: the GEMV's fp32 result (M, N) is not written to y (may be NULL) but stored over NVLink into
 *              slot `rank` of every rank's exchange buffer; the last CTA then raises this rank's flag there.
 *  gather = 1 (with NB_PRO_ADD_RMSNORM): delta is the sum, in rank order, of the vectors (M, K) the ranks
 *              pushed last; every CTA waits (bounded) for all flags.  All ranks compute the same bits.
 * Every rank owns one buffer of nb_exchange_buffer_bytes(world, max_count) bytes that all ranks can
 * address (peer-mapped, e.g. symmetric memory).  Set-up, once: zero-fill the buffer, call
 * nb_exchange_init(own buffer, peer_bufs, ...) where peer_bufs is a HOST array of `world` device
 * pointers, entry q = rank q's buffer as mapped into this process (entry `rank` = the own buffer; the
 * table is copied into the buffer, synchronously), then synchronise all ranks before the first push.
 * max_count >= M*N (push) and M*K (gather), a multiple of 4.  All ranks must issue the same sequence
 * of push and gather calls, and a push must be consumed (a gather by nb_gemv_tp or nb_exchange_gather)
 * before the next push.  A workspace is required (its status word receives NB_ERR_TIMEOUT when the
 * wait of spin_limit probes, 0 = default of several seconds, runs out; the kernel then continues with
 * what has arrived and does not hang, and later launches that find the status word set do not wait again).
 * Plain loads and stores on peer memory only: no TMA, no multicast.
 * nb_exchange_gather: the same sum written to out (count floats), for a consumer that is not a GEMV. */
size_t nb_exchange_buffer_bytes(int world, int max_count);
int nb_exchange_init(void* exchange, const uint64_t* peer_bufs, int world, int rank, int max_count);
int nb_gemv_tp(int prologue, const float* x, const float* delta, const float* norm_weight, float eps, float* x_out, int M,
               const uint8_t* packed, const void* codebook, int cb_dtype, int bits, int block_size, int N, int K, void* y,
               int y_dtype, void* workspace, size_t workspace_bytes, void* exchange, int world, int rank, int max_count,
               int gather, int push, uint32_t spin_limit, void* stream);
int nb_exchange_gather(float* out, int count, const void* exchange, int world, int rank, int max_count, uint32_t spin_limit,
                       int* status, void* stream);

/* ---- one-shot all-reduce (sum, fp32) over peer-mapped buffers, for the all-reduce after the
 * row-sharded projections of the tensor-parallel decoder (the reference has no multi-GPU inference;
 * NCCL all_reduce is the library equivalent).  Every rank owns one buffer of
 * nb_allreduce_buffer_bytes(world, max_count) bytes, zero-filled once, that all ranks can address
 * (peer-mapped, e.g. symmetric memory); peer_bufs is a HOST array of `world` device pointers, entry
 * q = rank q's buffer as mapped into this process.  count and max_count are multiples of 4, in and
 * out 16-byte aligned (in == out is allowed).  All ranks must issue the same sequence of calls.
 * Results are bit-identical on all ranks.  spin_limit = 0 selects the default bound of the wait for
 * the peers; when it runs out the kernel writes NB_ERR_TIMEOUT to *status (device int, may be NULL)
 * and returns without hanging. */
size_t nb_allreduce_buffer_bytes(int world, int max_count);
int nb_allreduce(const float* in, float* out, int count, const uint64_t* peer_bufs, int world, int rank,
                 int max_count, uint32_t spin_limit, int* status, void* stream);

/* ---- nb_gemv without a caller-provided workspace.  No counterpart in the reference.
 * For callers that cannot allocate device memory — a plugin that is handed only its input and
 * output buffers, code that runs while a stream is being captured or under a frozen memory
 * budget — the split-K scratch is a 4 MiB array built into the library's device image (every GPU
 * that loads the library holds it until the process exits).  Arguments are those of nb_gemv
 * minus the workspace.  Limits and rules:
 *  - shapes whose scratch need (nb_gemv_workspace_bytes) exceeds 4 MiB are refused with
 *    NB_ERR_WORKSPACE and a message in nb_last_cuda_error(); nothing is launched;
 *  - the first call on a device looks the array's address up (with that device current); make
 *    that first call before any stream capture begins;
 *  - the call enqueues a 16 KB clear of the array's head on `stream`, then the kernel; it calls no
 *    allocation or free routine of CUDA or of any library;
 *  - all calls on a device share the one array, which keeps the previous call's partial sums:
 *    two calls that overlap on the GPU (different streams, or graph branches) race.  Serialise
 *    them on one stream, or use nb_gemv with one workspace per stream. */
int nb_gemv_static(const void* x, int x_dtype, int M, const uint8_t* packed, const void* codebook, int cb_dtype,
                   int bits, int block_size, int N, int K, void* y, int y_dtype, void* stream);
/* Status word of the built-in array on the current device: *host_out = 0, or NB_ERR_TIMEOUT if a
 * bounded wait of any nb_gemv_static call ran out since the word was last cleared (clear != 0 resets
 * it).  Synchronises the device; no counterpart in the reference. */
int nb_gemv_static_status(int* host_out, int clear);

/* ---- persistent multi-matrix decode kernel ("stream" programs).
 * One launch runs a whole list of operations (a decode step: 26 x [qkv, attention, out_proj, gate_up,
 * down] + LM head + argmax; or any group of packed matvecs) on one CTA per SM, with the packed weights
 * streamed continuously through shared memory and device-side flags instead of kernel boundaries between
 * dependent operations.  Replaces the per-token launch sequence of inference/generate_torch.py:150-162
 * (forward) and :307-311 (greedy loop) and the per-call matvec of inference/cuda_kernel.py:38-104.
 *
 * Weights are read in a tile-major copy of the packed matrix, built once at load time by nb_stream_pack
 * from the nativebit/pack.py byte stream and the codebooks (the reference's JAX path re-orders blocks at
 * load time in the same spirit, nativebit_jax/packed_kernel.py:34-60).  row_mode 0 keeps the row order;
 * row_mode 1 expects a fused [gate | up] matrix of N rows and interleaves groups of 8 gate rows with the
 * matching 8 up rows, which the NB_SEPI_SWIGLU epilogue needs (N % 16 == 0).  The copy holds
 * nb_stream_packed_bytes(N, K, bits) bytes (same size as indices + fp16 codebooks, rows padded to 16);
 * codebooks are stored as fp16 (an fp32 codebook is rounded, as in nb_gemv).
 *
 * An operation is an nb_stream_op (160 bytes; unused fields zero).  Pointers are device pointers.
 *  NB_SOP_GEMV   y = W x.  p[0] stream-layout weights; i[0] N, i[1] K (multiple of 128, <= 7168), i[2] bits.
 *     prologue (how x is formed; i[3] = dtype of p[1] for NB_SPRO_VEC):
 *       NB_SPRO_VEC         x = p[1][0..K) (NB_F32 carried as two fp16 terms, NB_F16 / NB_BF16 as one)
 *       NB_SPRO_EMBED_NORM  h = table p[1] (bf16, i[13] rows; row *p[2] (int64), clamped to the table);
 *                           x = h * p[3] (K floats), result / rms(h)
 *       NB_SPRO_ADD_NORM    h += sum of i[5] slots of p[1] (floats, i[7] apart); then as above (f[0] = eps)
 *       NB_SPRO_ATTN_MERGE  x = attention output merged from the partials p[1] written by NB_SOP_ATTN:
 *                           i[9] heads, i[10] splits, i[11] head_dim, i[12] first column (others are zero)
 *       h is the residual stream; it lives in every CTA's shared memory for the whole launch.
 *     epilogue (where y goes, p[4]):
 *       NB_SEPI_STORE   y[n] of dtype i[4]                                   (needs NB_SOPF_ALIGN)
 *       NB_SEPI_SLOTS   fp32 partial sums: i[6] slots, i[8] floats apart; the consumer adds the slots.
 *                       i[6] >= nb_stream_slots(N, K, nb_stream_ctas())
 *       NB_SEPI_SWIGLU  fp32 act[c] = silu(gate_c) * up_c, N/2 values (row_mode 1 weights, NB_SOPF_ALIGN)
 *  NB_SOP_ATTN   RoPE + KV-cache write + single-query attention for one new token (inference/
 *     generate_torch.py:48-60, 86-97): p[0] qkv as i[5] slots i[7] apart ([q|k|v] of i[0] local heads),
 *     p[1]/p[2] cos/sin tables (ctx, head_dim) repeated per pair, p[3] position (int64), p[4]/p[5] key and
 *     value caches (heads, ctx, head_dim) fp32, p[6] partials out: (heads * splits) x (head_dim + 2) floats.
 *     i[1] head_dim (multiple of 4, <= 128), i[2] ctx, i[3] splits of the keys per head.
 *  NB_SOP_HEAD   final RMSNorm + tied LM head + soft-cap (generate_torch.py:157-159): p[0] bf16 table
 *     (i[0] rows, i[1] = C columns), p[1] last residual update as i[5] slots i[7] apart, p[3] norm weight,
 *     p[4] logits out (i[0] floats), p[5] candidates out (2 x CTAs words); f[0] eps, f[1] cap; i[8] = index of
 *     row 0 in the whole vocabulary.
 *  NB_SOP_ARGMAX token = lowest index among the largest candidates: p[0] candidates, i[0] their count,
 *     p[1] token out (int64), p[2] position (int64, incremented; may be NULL).
 *  NB_SOP_REDUCE y (p[4], dtype i[4], i[0] values) = sum of i[5] slots of p[1], i[7] floats apart.
 * flags: NB_SOPF_WAIT_PREV  the operation reads results of the operation before it: wait for all CTAs;
 *        NB_SOPF_ALIGN      split the rows between CTAs in whole 16-row tiles (no partial slots);
 *        NB_SOPF_REUSE_X    the activations staged by the previous NB_SOP_GEMV are used again.
 *
 * nb_stream_run takes the program twice: a host copy, which it validates, and the same bytes in device
 * memory, which the kernel reads.  `state` is nb_stream_state_bytes() of device memory, zero-filled once;
 * it carries the flag words, a sequence number that lets the launch be replayed from a CUDA graph, and a
 * status word (uint32 index 513) set to NB_ERR_TIMEOUT if a bounded wait ran out (the launch then finishes
 * without hanging; results are invalid).  One launch at a time per state buffer.  The launch is cooperative
 * (all nb_stream_ctas() CTAs resident).  All packed matrices of a program share one `bits`.
 * Limits: at most nb_stream_max_ops() operations; one activation row (batch 1); K <= 7168; the norm prologues and
 * the head need a model width <= 2560; fewer than 65536 (16-row x 128-weight) units per matrix. */
typedef enum { NB_SOP_GEMV = 1, NB_SOP_ATTN = 2, NB_SOP_HEAD = 3, NB_SOP_ARGMAX = 4, NB_SOP_REDUCE = 5 } nb_stream_kind;
typedef enum { NB_SPRO_VEC = 0, NB_SPRO_EMBED_NORM = 1, NB_SPRO_ADD_NORM = 2, NB_SPRO_ATTN_MERGE = 3 } nb_stream_prologue;
typedef enum { NB_SEPI_STORE = 0, NB_SEPI_SLOTS = 1, NB_SEPI_SWIGLU = 2 } nb_stream_epilogue;
enum { NB_SOPF_WAIT_PREV = 1, NB_SOPF_ALIGN = 2, NB_SOPF_REUSE_X = 4 };
typedef struct {
  int32_t kind, flags, pro, epi;
  void* p[8];
  int32_t i[16];
  float f[4];
} nb_stream_op;
size_t nb_stream_packed_bytes(int N, int K, int bits);
int nb_stream_pack(const uint8_t* packed, const void* codebook, int cb_dtype, int bits, int N, int K, int row_mode,
                   uint8_t* out, void* stream);
size_t nb_stream_state_bytes(void);
int nb_stream_max_ops(void);
int nb_stream_ctas(void);
int nb_stream_slots(int N, int K, int ctas);
int nb_stream_run(const nb_stream_op* ops_host, const nb_stream_op* ops_device, int n_ops, void* state, uint32_t spin_limit,
                  void* stream);

/* ---- a group of INDEPENDENT packed matvecs in one launch (none reads another's output): y_i = W_i x_i for one
 * activation vector each.  The reference runs one launch per matrix (inference/triton_kernel.py:240-256,
 * inference/cuda_kernel.py:84-104); here the row tiles of all matrices form one sequence that the CTAs share
 * by weight bytes, a warp computes a whole 16-row tile from the first k-block to the last with the sums in
 * registers, and nothing waits on anything but its own copies (no flags, no status word needed).
 * Weights are nb_stream_pack copies (row_mode 0), all of one `bits`; x: m rows of k values of x_dtype, 16-byte
 * aligned, K % 128 == 0 and K <= 7168 (one row: NB_F32 is carried as two fp16 terms; 2..8 rows: NB_F16 or
 * NB_BF16 only, each row one column of the MMA); y: m rows of n values of y_dtype.  At most
 * nb_group_max_items() matvecs and 6 distinct activation matrices whose staged copies fit 104 KB of shared
 * memory (64 KB at 4 bits; a row takes K * 2.5 bytes per fp16 term, the first term of an fp32 vector 17920
 * bytes; beyond 64 KB the copy rings are one stage shorter).
 * nb_group_build validates the list and writes the launch plan (nb_group_plan_bytes(items, n) bytes: a header
 * and one word per 16-row tile) into host memory: the row tiles are dealt out to the CTAs longest first, each
 * to the CTA with the least work so far, so that all CTAs finish within one short tile of one another.  The
 * caller copies the plan to device memory once and passes both copies to nb_group_run (the host copy for the
 * launch geometry).  Results are bit-identical from run to run. */
typedef struct {
  const void* w;
  const void* x;
  void* y;
  int32_t n, k, x_dtype, y_dtype;
  int32_t m;          /* activation rows, 1..8 (0 means 1): x is (m, k), y is (m, n), both row-major */
  int32_t reserved;   /* zero */
} nb_group_item;
size_t nb_group_plan_bytes(const nb_group_item* items, int n_items);
int nb_group_max_items(void);
int nb_group_build(const nb_group_item* items, int n_items, int bits, void* plan_out, size_t plan_bytes);
int nb_group_run(const void* plan_device, const void* plan_host, void* stream);

/* ---- one packed matvec of a chain of dependent launches (the decode step at one sequence), over the
 * nb_stream_pack copy of the weights: y (N fp32) = W . act(x).  Same contract as nb_gemv_fused at M = 1
 * (inference/triton_kernel.py:240-256 with the element-wise step of inference/generate_torch.py:109-117 in front):
 * prologue NB_PRO_NONE: act = x (K values of x_dtype; NB_F32 carried as two fp16 terms);
 * NB_PRO_ADD_RMSNORM: x fp32 residual, delta (K, may be NULL) added first, act = rmsnorm(x + delta) * norm_weight,
 * x + delta written to x_out (may be NULL; must not alias x); NB_PRO_SILU_MUL: x = [gate | up] (2K fp32),
 * act = silu(gate) * up.  One CTA per SM; the k-blocks of a 16-row tile are shared by a team of warps of one CTA, so
 * there is no workspace and nothing to wait for but the launch's own copies; weights are requested before the
 * launch waits for the one before it (programmatic dependent launch).  K % 128 == 0, K <= 7168; 16-byte aligned
 * pointers.  swiglu is a set of flags.  Bit 0: W is a fused [gate | up] matrix packed with nb_stream_pack row_mode 1
 * (N % 16 == 0) and y receives the N / 2 values silu(gate_c) * up_c (the SwiGLU of generate_torch.py:116-117 in the
 * epilogue).  Bit 1: fp32 activations enter the tensor cores rounded to ONE fp16 term (11 significant bits) instead of
 * two (22 bits): half the tensor-core instructions, an error of a few 1e-4 of max |y| per matvec — measured 4e-3 of
 * max |logit| at the end of the 26-layer decoder, above its 2e-3 gate, so it is off in this package's decode session.
 * Bit 2 (not with bit 0): y += W . act(x) — the residual update of a decoder block (generate_torch.py:114, :117) inside the
 * matvec that produces it; every output is read and written by the same thread.  Bit-identical from run to run. */
int nb_gemv_stream(int prologue, const void* x, int x_dtype, const float* delta, const float* norm_weight, float eps,
                   float* x_out, const uint8_t* w_stream, int bits, int N, int K, float* y, int swiglu, void* stream);
/* nb_gemv_stream for M = 1 .. nb_gemv_stream_max_rows(bits, K) fp32 activation rows (a decode step of a few sequences,
 * inference/generate_torch.py:307-311 with a batch): ONE pass over the weights, the rows ride in the columns of the
 * tensor-core instructions that a single row leaves empty.  x (M, K) — (M, 2K) rows [gate | up] with NB_PRO_SILU_MUL —,
 * delta and x_out (M, K), y (M, N) fp32, all row-major and 16-byte aligned.  The row limit is what the staged rows
 * leave of the shared memory (8 rows at K = 2560, 3 at K = 6912); a caller with more rows splits them over calls.
 * swiglu = 1: the SwiGLU epilogue of nb_gemv_stream (row_mode 1 copy of [gate | up]), y is (M, N / 2). */
int nb_gemv_stream_max_rows(int bits, int K);
int nb_gemv_stream_rows(int prologue, const float* x, int M, const float* delta, const float* norm_weight, float eps,
                        float* x_out, const uint8_t* w_stream, int bits, int N, int K, float* y, int swiglu, void* stream);

/* Launch geometry nb_gemv will use for a shape on the current device (no launch; works without
 * a GPU, assuming 148 SMs): out6 = {grid.x, grid.y (k partitions), threads per CTA, dynamic
 * shared memory bytes, row tiles per CTA, k-groups per partition}.  No counterpart in the
 * reference; used for reporting and tests. */
int nb_gemv_plan(int M, int N, int K, int bits, int block_size, int cb_dtype, int* out6);

#ifdef __cplusplus
}
#endif
#endif /* NATIVEBIT_B200_H_ */
