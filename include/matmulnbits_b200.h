/* C ABI of the B200 (sm_100a) MatMulNBits library.
 *
 * This is the thin layer between the C++ operator class (MatMulNBitsKernel, the
 * counterpart of the reference's KernelBase subclasses) and the hand-written CUDA kernels.
 * Signatures use plain pointers and sizes only. Every function returns 0 on success and a
 * non-zero mnb_status otherwise; mnb_last_error() gives the message of the calling thread's
 * last failure. Nothing here throws, and nothing falls back to the CPU: without a CUDA
 * device every compute entry point fails with MNB_ERR_CUDA.
 *
 * Operator contract (com.microsoft.MatMulNBits, fp32 activations):
 *   B       uint8 [N, n_blocks, block_size*bits/8], n_blocks = ceil(K/block_size); element
 *           2i of a 4-bit blob is the LOW nibble of byte i (the reference's packed-INT4
 *           convention, onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.h:42-47)
 *   scales  fp32 [N*n_blocks]
 *   zero_points (optional) packed like B, one code per block, rows padded to a whole byte;
 *           default 2^(bits-1)
 *   bias    (optional) fp32 [N]
 *   Y[m,n] = sum_k A[m,k] * (q[n,k] - zp[n,k/block_size]) * scale[n,k/block_size] + bias[n]
 */
#ifndef MATMULNBITS_B200_H_
#define MATMULNBITS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum mnb_status {
  MNB_OK = 0,
  MNB_ERR_INVALID_ARGUMENT = 1, /* maps to std::invalid_argument in the C++ operator class */
  MNB_ERR_CUDA = 2,             /* maps to std::runtime_error */
  MNB_ERR_UNSUPPORTED = 3,
  MNB_ERR_DEVICE_TIMEOUT = 4    /* a bounded device-side wait gave up; context still usable */
} mnb_status;

/* Which kernel family runs. AUTO picks by M, bits, block_size and accuracy_level and always finds a kernel
 * for a valid node: shapes none of the families below takes (block_size 16, rows of any length, odd sizes)
 * run on word-wise CUDA-core kernels; 8-bit weights with 5 <= M <= 16 run on integer tensor cores. */
typedef enum mnb_path {
  MNB_PATH_AUTO = 0,
  MNB_PATH_GEMV = 1,    /* CUDA-core fused unpack-dequant GEMV, fp32 accumulate (decode) */
  MNB_PATH_TCGEN05 = 2, /* TMA + smem dequant to bf16 + tcgen05/TMEM MMA (prefill), 128 weight rows per CTA */
  MNB_PATH_INT8 = 3,    /* accuracy_level 4: per-block int8 A, int32 block dots */
  MNB_PATH_GEMV_MMA = 4, /* decode on warp-level MMA, exact two-piece fp16 split of A */
  MNB_PATH_TCGEN05_WIDE = 5, /* prefill, tiles of 512 rows x up to 256 tokens on pairs of CTAs for any M (AUTO picks them for M > 16 when they pay) */
  MNB_PATH_INT8_MMA = 6, /* accuracy_level 4 on integer tensor-core MMA (AUTO picks it when the shape fits) */
  MNB_PATH_GEMV_MMA_MULTI = 7, /* decode on warp-level MMA, several column tiles of tokens per pass */
  MNB_PATH_GEMV_IMMA = 8, /* decode on integer MMA, A as three base-128 digits (block_size >= 128; AUTO picks it for M <= 2) */
  MNB_PATH_GEMV_DIGITS = 9, /* decode, accuracy_level 0: three digit rows per token through the sixteen-row integer-MMA kernel */
  MNB_PATH_GEMV_DIRECT = 10, /* decode on integer MMA with the weights streamed from global memory straight into each warp
                               (no staging ring), M <= 2, block_size 128; AUTO's choice for M = 1 where the resident kernel does not fit */
  MNB_PATH_GEMV_RESIDENT = 11 /* decode of one token on integer MMA: a producer warp asks the TMA unit for the CTA's whole
                                 share of the weights at kernel start; block_size 128 or 32; AUTO's first choice for M = 1 */
} mnb_path;

/* Device-resident, immutable weights of one MatMulNBits node. Plays the role the reference
 * gives its per-node plan cache (onnx_light_cpu/kernels/math/gemm_kernel.cc:100-184): built
 * once per node from the initializer tensors, reused by every Run. */
typedef struct mnb_weights mnb_weights;

/* Message of the last failure on the calling thread (never NULL). */
const char *mnb_last_error(void);

/* Number of CUDA devices visible; 0 with MNB_OK when the driver reports none. */
int mnb_device_count(int *count);

/* Library identification: "matmulnbits_b200 <version> sm_100a". */
const char *mnb_version(void);

/* Uploads one node's constant operands from HOST memory to `device`.
 * Replaces: the per-call operand packing of IntegerMatMul4Bit2D
 * (onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:164-206) with a one-time
 * constant-weight upload. zero_points and bias may be NULL. */
int mnb_weights_create(int device, const uint8_t *b, const float *scales,
                       const uint8_t *zero_points, const float *bias, int64_t n, int64_t k,
                       int bits, int block_size, mnb_weights **out);

/* Same, but the four operand pointers are DEVICE pointers that the caller keeps alive; no
 * copy is made. Used by benchmarks and by sharded callers that fill device memory directly. */
int mnb_weights_wrap_device(int device, const uint8_t *b, const float *scales,
                            const uint8_t *zero_points, const float *bias, int64_t n, int64_t k,
                            int bits, int block_size, mnb_weights **out);

int mnb_weights_destroy(mnb_weights *weights);

/* Bytes the operator must read and write once per call (weights + scales + zero points +
 * bias + A + Y): the algorithmic traffic used for roofline figures. */
int64_t mnb_algorithmic_bytes(int64_t m, int64_t n, int64_t k, int bits, int block_size,
                              int has_zero_points, int has_bias);

/* Y = MatMulNBits(A) with A and Y in HOST memory. Synchronous: copies A to the device,
 * runs the selected kernel, copies Y back and waits.
 * Replaces: the body of a KernelBase::operator() that calls IntegerMatMul2D on host
 * tensors (onnx_light_cpu/kernels/math/integer_matmul_kernel.cc:298-339). */
int mnb_matmul_host(mnb_weights *weights, const float *a_host, int64_t m, int accuracy_level,
                    int path, float *y_host);

/* Y = MatMulNBits(A) with A and Y in DEVICE memory, asynchronous on `stream`
 * (a cudaStream_t passed as void*, NULL = default stream).
 * Replaces: IntegerMatMul4Bit2D's raw-pointer entry point
 * (onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.h:52-55). */
int mnb_matmul_device(mnb_weights *weights, const float *a_dev, int64_t m, int accuracy_level,
                      int path, float *y_dev, void *stream);

/* Sibling nodes in one call: `count` (1..MNB_MAX_GROUPED_NODES) nodes that take the SAME
 * activations - the q / k / v or the gate / up projections of a decoder layer - write
 * y_dev[i] = MatMulNBits_i(A), each a dense row-major [m, N_i] device matrix. Same K and same GPU
 * for all nodes, no node or output twice. What the nodes share is done once and the nodes' row
 * tiles form one sequence over the CTAs of a single kernel launch: at M = 1 (accuracy_level 0,
 * 4-bit, block_size 128) one kernel streams all nodes' weights behind activations staged once; at
 * accuracy_level 4 the activations are quantized once and one integer-MMA launch covers the
 * group; for 5..16 tokens at accuracy_level 0 the digit rows are made once and one launch of the
 * one-pass digit kernel covers the group. Any other group runs node by node with
 * the same results as separate mnb_matmul_device calls. Asynchronous on `stream`; bounded waits
 * of a grouped launch report through handles[0] (mnb_weights_poll_status).
 * Replaces: the consecutive MatMul nodes over one input that the reference's graph runs one by
 * one (q/k/v and gate/up of docs/next_steps/2026/2026_08_qwen3_inference.rst:374-380). */
#define MNB_MAX_GROUPED_NODES 3
int mnb_matmul_device_group(mnb_weights *const *handles, int count, const float *a_dev, int64_t m,
                            int accuracy_level, float *const *y_dev, void *stream);

/* Column-sharded form: writes this shard's N columns into a row-major [m, ld_y] matrix
 * starting at column `col_offset`, so g shards tile one [m, g*N] output. */
int mnb_matmul_device_strided(mnb_weights *weights, const float *a_dev, int64_t m,
                              int accuracy_level, int path, float *y_dev, int64_t ld_y,
                              int64_t col_offset, void *stream);

/* Column gather without a collective ----------------------------------------------------------
 * For a node sharded by output column over the GPUs of one box, each rank can store its columns
 * straight into every rank's gathered result through peer-mapped memory instead of running an
 * all-gather afterwards. No counterpart in the reference (a CPU library has no such step); the
 * closest notion is the N split of onnx_light_cpu/impl/math/gemm_kernel.cc:1219-1258, whose
 * threads write disjoint column ranges of one shared Y.
 *
 * mnb_peer_buffer_create allocates `bytes` of device memory (zero filled) that other processes
 * of the box can map, and writes its inter-process handle (MNB_IPC_HANDLE_BYTES bytes, to be
 * sent to the peers by any host channel). mnb_peer_buffer_open maps a peer's buffer into this
 * process and enables peer access; _close unmaps it; _destroy frees an own buffer. */
#define MNB_IPC_HANDLE_BYTES 64
#define MNB_MAX_GATHER_RANKS 8
int mnb_peer_buffer_create(int device, size_t bytes, void **dev_ptr, unsigned char *handle_out);
int mnb_peer_buffer_open(int device, const unsigned char *handle, void **peer_ptr);
int mnb_peer_buffer_close(int device, void *peer_ptr);
int mnb_peer_buffer_destroy(int device, void *dev_ptr);

/* Product whose [m, N] result is stored at the same window (ld_y, col_offset) of `ranks` buffers:
 * y_ranks[r] is rank r's gathered result as mapped in this process (y_ranks[rank] is the local
 * one). Decode shapes of the tensor-core decode kernels (accuracy_level 0, M <= 16, 4-bit) store
 * to every buffer from the kernel itself; every other shape (8-bit weights, more tokens,
 * accuracy_level 4) runs through the ordinary dispatch into the local window, which one more
 * kernel then copies to the peers. Either way each CTA pushes its part of the window to the
 * peers with coalesced stores as it finishes, and the last CTA to finish sets
 * flags_ranks[r][rank] = epoch on every rank ("my columns of this step are stored"): no separate
 * kernel. With `wait` non-zero that CTA then waits, bounded, until the local
 * flags_ranks[rank][0..ranks) all carry the epoch, so that the result is complete when the stream
 * has passed the call. A rank's flag for one call implies its earlier calls (every rank makes the
 * same sequence of calls), so a run of nodes needs the wait on its last node only, or none and
 * one mnb_gather_wait where the gathered results are first read: consecutive nodes then do not
 * each pay a round trip
 * between GPUs. `epoch` must grow by one per step on all ranks, or be 0 on all ranks and all
 * steps: then the step number is kept on the device in flags_ranks[rank][MNB_MAX_GATHER_RANKS]
 * and incremented by the call itself, which is what a captured and replayed CUDA graph needs.
 * Each flags array holds at least MNB_MAX_GATHER_RANKS + 1 ints, zero at start. Every rank must
 * make the same sequence of calls. A wait that gives up sets the status word
 * (mnb_weights_poll_status).
 * mnb_matmul_device_gather is the accuracy_level 0, wait = 1 form. */
int mnb_matmul_device_gather_ex(mnb_weights *weights, const float *a_dev, int64_t m, int accuracy_level,
                                float *const *y_ranks, int *const *flags_ranks, int ranks, int rank,
                                int64_t ld_y, int64_t col_offset, int epoch, int wait, void *stream);
int mnb_matmul_device_gather(mnb_weights *weights, const float *a_dev, int64_t m,
                             float *const *y_ranks, int *const *flags_ranks, int ranks, int rank,
                             int64_t ld_y, int64_t col_offset, int epoch, void *stream);

/* Waits (one small kernel on `stream`, bounded, status word of `weights`) until each of the
 * `count` LOCAL flag arrays carries its epoch for all `ranks` ranks; epochs == NULL or an epoch of
 * 0 means the step this rank itself published last through that array (self-counting mode). */
#define MNB_MAX_GATHER_WAITS 8
int mnb_gather_wait(mnb_weights *weights, int *const *flags_local, const int *epochs, int count, int ranks,
                    void *stream);

/* Waits for the device and reads the status word that kernels with bounded waits write when
 * they give up (0 = fine, see MNB_ERR_DEVICE_TIMEOUT). Clears it after reading. The
 * host-buffer call checks it itself; callers of the asynchronous entry points use this. */
int mnb_weights_poll_status(mnb_weights *weights, int *status);

/* Parity hooks (device pointers) ---------------------------------------------------------- */

/* out[n*K + k] = q[n,k] - zp[n,k/block_size] as int32: the integer dequantization that must
 * be bit-exact (integer_gemm_vnni.cc:60-93 nibble order, :208-223 exact integers). */
int mnb_dequant_int_device(mnb_weights *weights, int32_t *out_dev, void *stream);

/* accuracy_level 4 stage 1: per (row, block) scale = max|A|/127, aq = clamp(rne(A/scale)).
 * A block that holds a NaN or an infinity gets scale NaN and codes 0: every output of that token
 * is then NaN, like at accuracy_level 0 (a NaN is not clamped to -127 behind the caller's back). */
int mnb_quantize_a_device(const float *a_dev, int64_t m, int64_t k, int block_size,
                          int8_t *aq_dev, float *a_scales_dev, void *stream);

/* accuracy_level 4 stage 2 exposed: dots[(m*N+n)*n_blocks+blk] = sum aq*(q-zp), int32 exact
 * (the same modulo-2^32 integer semantics as IntegerDotU8S8Scalar,
 * integer_gemm_vnni.cc:48-56). */
int mnb_int8_block_dots_device(mnb_weights *weights, const int8_t *aq_dev, int64_t m,
                               int32_t *dots_dev, void *stream);

/* The same block dots, but produced by the production integer-MMA kernel of accuracy_level 4 itself
 * (an instrumented instantiation of it: same fragment layout, swizzled tiles, signed-code form and
 * zero-point correction, plus a store of every block sum before it is scaled). A is quantized on
 * the device exactly as mnb_matmul_device(accuracy_level = 4) does it; y_dev [m, N] receives the
 * ordinary result, dots_dev [m, N, n_blocks] the sums (cleared by the call). m <= 8 and a shape
 * the integer-MMA kernel takes, else MNB_ERR_UNSUPPORTED. Exactness to compare with:
 * IntegerDotU8S8Scalar, onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:48-56. */
int mnb_int8_mma_block_dots_device(mnb_weights *weights, const float *a_dev, int64_t m, float *y_dev,
                                   int32_t *dots_dev, void *stream);

/* accuracy_level-4 product Y = MatMulNBits(A) that allocates nothing. It has no counterpart in
 * the reference. It is meant for callers that are not allowed to reach cudaMalloc while they
 * run: a serving loop whose steady state must stay free of the device-wide synchronisation and
 * the possible out-of-memory failure of an allocation, or a host that owns all device memory
 * itself and gives a plug-in none. mnb_matmul_device(accuracy_level = 4) grows cudaMalloc'ed
 * scratch for the quantized activations; this entry point keeps them in an array that is part
 * of the library image instead (about 0.3 MB on every GPU that loads the library, held until
 * the process exits).
 *   - limits: 1 <= m <= MNB_STATIC_MAX_TOKENS and ceil(K/block_size)*block_size <=
 *     MNB_STATIC_MAX_PADDED_K; anything larger is refused with MNB_ERR_INVALID_ARGUMENT;
 *   - a_dev [m, K] and y_dev [m, N] are device pointers of the GPU that holds the weights (plain
 *     host memory or another GPU's memory is refused with MNB_ERR_INVALID_ARGUMENT, as by the
 *     other device-pointer entry points); the work is queued on `stream`, the quantization and
 *     the product of a call as a pair, also against calls from other host threads;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress with that device current); make that first call outside any
 *     stream capture;
 *   - all calls share the one array. It keeps the previous call's bytes; every byte a call
 *     reads it first rewrites itself, so nothing needs clearing, but two calls whose kernels
 *     overlap on the GPU (different streams, different handles) would race on it: keep calls
 *     to this entry point ordered on the device. */
#define MNB_STATIC_MAX_TOKENS 16
#define MNB_STATIC_MAX_PADDED_K 16384
int mnb_matmul_int8_static(mnb_weights *weights, const float *a_dev, int64_t m, float *y_dev,
                           void *stream);

/* Number of kernels this library has launched in the calling process (for benchmarks). */
int64_t mnb_launch_count(void);

/* Name of the kernel the last mnb_matmul_* call on this thread dispatched to. */
const char *mnb_last_kernel(void);

/* Geometry accessors. */
int64_t mnb_weights_n(const mnb_weights *weights);
int64_t mnb_weights_k(const mnb_weights *weights);
int mnb_weights_bits(const mnb_weights *weights);
int mnb_weights_block_size(const mnb_weights *weights);

#ifdef __cplusplus
}
#endif

#endif /* MATMULNBITS_B200_H_ */
