// C ABI of the library (declarations and contract: include/matmulnbits_b200.h).
// Owns the per-node device weight handle, scratch buffers and the dispatch between kernels.
// No CPU fallback exists: every compute entry point needs a CUDA device.

#include "../../include/matmulnbits_b200.h"

#include "nbits_common.cuh"

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>

namespace mnb {

namespace {
std::atomic<std::int64_t> g_launches{0};
thread_local std::string t_last_error = "";
thread_local const char *t_last_kernel = "";
} // namespace

void CountLaunch(int launches) { g_launches.fetch_add(launches, std::memory_order_relaxed); }

int WantedProducers(int kernel_default) { return kernel_default; }

thread_local bool t_dependent_launch_hint = false;
void SetDependentLaunchHint(bool allowed) { t_dependent_launch_hint = allowed; }
bool DependentLaunchHint() { return t_dependent_launch_hint; }

// out[n*K + k] = q - zp, one thread per element.
__global__ void __launch_bounds__(256)
    nbits_dequant_int_kernel(const WeightView w, std::int32_t *out) {
  const std::int64_t total = w.n * w.k;
  for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<std::int64_t>(gridDim.x) * blockDim.x) {
    const std::int64_t row = i / w.k;
    const std::int64_t kk = i - row * w.k;
    out[i] = CodeOf(w, row, kk) - ZeroPointOf(w, row, static_cast<int>(kk / w.block_size));
  }
}

const char *LaunchDequantInt(const WeightView &w, std::int32_t *out, cudaStream_t stream) {
  const std::int64_t total = w.n * w.k;
  if (total <= 0) {
    return nullptr;
  }
  std::int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) {
    blocks = 148 * 16;
  }
  nbits_dequant_int_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(w, out);
  if (cudaGetLastError() != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return "nbits_dequant_int_kernel";
}

} // namespace mnb

using mnb::OutputView;
using mnb::WeightView;

struct mnb_weights {
  WeightView view{};
  int device = 0;
  int sm_count = 148;
  bool owns = false;
  void *owned[4] = {nullptr, nullptr, nullptr, nullptr};
  // status word of the bounded device-side waits: page-locked host memory (`status_host`) and its
  // device alias (`status_dev`), so reading it after a synchronize needs no copy
  int *status_dev = nullptr;
  int *status_host = nullptr;
  void *meta_dev = nullptr; // prepared scales / zero points for the MMA decode kernel
  void *zp16_dev = nullptr; // prepared zero-point bytes for the direct-stream decode kernel
  unsigned *arrivals_dev = nullptr; // finished-CTA counter of the fused gather (zero between launches)
  // scratch, grown on demand (guarded by `mutex`)
  std::mutex mutex;
  void *scratch_a = nullptr; // bf16 activations (prefill) or int8 activations (accuracy_level 4)
  std::size_t scratch_a_bytes = 0;
  void *scratch_s = nullptr; // activation block scales (accuracy_level 4)
  std::size_t scratch_s_bytes = 0;
  // host-call staging
  float *a_dev = nullptr;
  float *y_dev = nullptr;
  std::size_t a_dev_bytes = 0;
  std::size_t y_dev_bytes = 0;
  cudaStream_t stream = nullptr;
  // last (A, Y) pair of the device-pointer entry points whose location has been checked
  const void *checked_a = nullptr;
  const void *checked_y = nullptr;
  // last (A, Y) pair of the host-buffer entry point and what the runtime said about it: the
  // device aliases of page-locked buffers (nullptr = stage through device memory)
  const void *host_a = nullptr;
  const void *host_y = nullptr;
  std::size_t host_a_bytes = 0;
  std::size_t host_y_bytes = 0;
  const float *host_a_alias = nullptr;
  float *host_y_alias = nullptr;
};

namespace {

int Fail(int code, const std::string &message) {
  mnb::t_last_error = message;
  return code;
}

int FailCuda(const char *what, cudaError_t err) {
  return Fail(MNB_ERR_CUDA, std::string("matmulnbits_b200: ") + what + ": " + cudaGetErrorString(err));
}

bool ValidGeometry(std::int64_t n, std::int64_t k, int bits, int block_size, std::string *why) {
  if (n <= 0 || k <= 0) {
    *why = "MatMulNBits requires positive N and K.";
    return false;
  }
  if (bits != 4 && bits != 8) {
    *why = "MatMulNBits supports bits = 4 or 8.";
    return false;
  }
  if (block_size < 16 || (block_size & (block_size - 1)) != 0) {
    *why = "MatMulNBits block_size must be a power of two >= 16.";
    return false;
  }
  return true;
}

void FillView(WeightView *v, std::int64_t n, std::int64_t k, int bits, int block_size) {
  v->n = n;
  v->k = k;
  v->bits = bits;
  v->block_size = block_size;
  v->n_blocks = static_cast<int>((k + block_size - 1) / block_size);
  v->blob_bytes = block_size * bits / 8;
  v->row_bytes = v->n_blocks * v->blob_bytes;
  v->zp_row_bytes = (v->n_blocks * bits + 7) / 8;
}

int SetupCommon(mnb_weights *h) {
  cudaError_t err = cudaSetDevice(h->device);
  if (err != cudaSuccess) {
    return FailCuda("cudaSetDevice", err);
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, h->device) == cudaSuccess && sms > 0) {
    h->sm_count = sms;
  }
  err = cudaHostAlloc(reinterpret_cast<void **>(&h->status_host), sizeof(int), cudaHostAllocMapped);
  if (err != cudaSuccess) {
    return FailCuda("cudaHostAlloc(status)", err);
  }
  *h->status_host = 0;
  err = cudaHostGetDevicePointer(reinterpret_cast<void **>(&h->status_dev), h->status_host, 0);
  if (err != cudaSuccess) {
    return FailCuda("cudaHostGetDevicePointer(status)", err);
  }
  err = cudaMalloc(&h->arrivals_dev, sizeof(unsigned));
  if (err == cudaSuccess) {
    err = cudaMemset(h->arrivals_dev, 0, sizeof(unsigned));
  }
  if (err != cudaSuccess) {
    return FailCuda("cudaMalloc(arrival counter)", err);
  }
  err = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
  if (err != cudaSuccess) {
    return FailCuda("cudaStreamCreate", err);
  }
  return MNB_OK;
}

// Builds the task-major scales / zero-point array once per node (constant-weight policy).
int PrepareMeta(mnb_weights *h) {
  if (mnb::DecodeDirectWantsZeroPointBytes(h->view)) {
    // one byte per block (16 x the zero point): rides the same asynchronous copies as the scales
    cudaError_t err = cudaMalloc(&h->zp16_dev, static_cast<std::size_t>(h->view.n) * h->view.n_blocks);
    if (err != cudaSuccess) {
      return FailCuda("cudaMalloc(zero-point bytes)", err);
    }
    if (!mnb::LaunchExpandZeroPoints(h->view, static_cast<unsigned char *>(h->zp16_dev), h->stream)) {
      return FailCuda("prepare zero-point bytes", cudaGetLastError());
    }
    err = cudaStreamSynchronize(h->stream);
    if (err != cudaSuccess) {
      return FailCuda("prepare zero-point bytes", err);
    }
    h->view.zp16 = static_cast<const unsigned char *>(h->zp16_dev);
  }
  const mnb::MetaGeometry geo = mnb::MetaGeometryOf(h->view);
  if (geo.bytes == 0) {
    return MNB_OK; // geometry not taken by the MMA decode kernel
  }
  cudaError_t err = cudaMalloc(&h->meta_dev, geo.bytes);
  if (err != cudaSuccess) {
    return FailCuda("cudaMalloc(meta)", err);
  }
  if (!mnb::LaunchPrepareMeta(h->view, static_cast<unsigned char *>(h->meta_dev), h->stream)) {
    return FailCuda("prepare meta", cudaGetLastError());
  }
  err = cudaStreamSynchronize(h->stream);
  if (err != cudaSuccess) {
    return FailCuda("prepare meta", err);
  }
  h->view.meta = static_cast<const unsigned char *>(h->meta_dev);
  return MNB_OK;
}

int Grow(void **ptr, std::size_t *have, std::size_t need) {
  if (need <= *have) {
    return MNB_OK;
  }
  if (*ptr != nullptr) {
    cudaFree(*ptr);
    *ptr = nullptr;
    *have = 0;
  }
  cudaError_t err = cudaMalloc(ptr, need);
  if (err != cudaSuccess) {
    return FailCuda("cudaMalloc(scratch)", err);
  }
  *have = need;
  return MNB_OK;
}

// Copies a small page-locked host buffer into device memory with a kernel: a kernel behind a
// kernel starts sooner than a kernel behind a copy-engine transfer, and the bytes of a decode
// step (M x K floats) cross the host link in a microsecond or two.
__global__ void __launch_bounds__(256) nbits_fetch_kernel(const uint4 *src, uint4 *dst, int count16,
                                                          const float *src_tail, float *dst_tail, int tail) {
  // a kernel launched behind this one with programmatic serialization may start at once; it
  // waits for this grid before it touches `dst`
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count16) {
    dst[i] = src[i];
  }
  if (i < tail) {
    dst_tail[i] = src_tail[i];
  }
}

// Waiting half of a gathered step, as a kernel of its own so that a caller can put it where the
// gathered result is first needed: warp i waits, bounded, until the local flag array i carries
// its epoch for every rank (epoch 0: the step count this rank itself published last).
struct GatherWaitList {
  int *flags[MNB_MAX_GATHER_WAITS];
  int epoch[MNB_MAX_GATHER_WAITS];
  int count;
  int ranks;
};

__global__ void __launch_bounds__(32 * MNB_MAX_GATHER_WAITS) nbits_gather_wait_kernel(GatherWaitList list, int *status) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= list.count) {
    return;
  }
  int epoch = list.epoch[warp];
  if (epoch == 0) {
    epoch = *reinterpret_cast<volatile int *>(list.flags[warp] + mnb::kMaxGatherRanks);
  }
  mnb::WaitStep(list.flags[warp], list.ranks, epoch, lane, status);
}

// Gathered step of a product that only wrote the local window (any kernel of the dispatcher): the
// window [m, n] is copied to the same place of every peer's buffer with plain stores, then the
// last CTA publishes the flags like the decode kernels do.
__global__ void __launch_bounds__(256)
    nbits_gather_push_kernel(mnb::OutputView out, std::int64_t m, std::int64_t n, int vector, mnb::GatherTail tail,
                             int *status) {
  // launched with programmatic stream serialization behind the kernels of the product: its blocks
  // may be resident early, the window is read once those kernels have completed
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const std::int64_t stride = static_cast<std::int64_t>(gridDim.x) * 256;
  const std::int64_t first = static_cast<std::int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (vector != 0) {
    const std::int64_t n4 = n / 4;
    for (std::int64_t i = first; i < m * n4; i += stride) {
      const std::int64_t row = i / n4;
      const std::int64_t at = row * out.ld + out.col_offset + (i - row * n4) * 4;
      const float4 v = *reinterpret_cast<const float4 *>(out.y + at);
      for (int r = 0; r < tail.n_peers; ++r) {
        *reinterpret_cast<float4 *>(tail.peers[r] + at) = v;
      }
    }
  } else {
    for (std::int64_t i = first; i < m * n; i += stride) {
      const std::int64_t row = i / n;
      const std::int64_t at = row * out.ld + out.col_offset + (i - row * n);
      const float v = out.y[at];
      for (int r = 0; r < tail.n_peers; ++r) {
        tail.peers[r][at] = v;
      }
    }
  }
  mnb::PublishWhenGridDone(tail, static_cast<int>(threadIdx.x), 256, 1, gridDim.x, status);
}

// AUTO sends at most this many tokens to the integer-digit decode kernel (two tokens per pass).
constexpr std::int64_t kImmaAutoTokens = 2;

// Token counts that AUTO sends to the one-pass digit kernel (nbits_digits_mma_kernel), by block size.
bool DigitSlicesWanted(const WeightView &w, std::int64_t m) {
  if (w.bits != 4 || m > 16) {
    return false;
  }
  // from five tokens on; from three on rows of 8192 k and more, where the fp16 kernels need several
  // passes or do not fit (K = 14336, M = 3 / 4, us per node: block 32 N = 4096 25.2 / 25.5 against
  // 31.5 / 33.2, N = 14336 62.3 / 62.5 against 82.3 / 83.6; block 128 N = 14336 49.6 / 50.1 against 68.9
  // and, at M = 4, no tensor-core kernel at all: 1.8 ms on the generic one)
  return m >= 5 || (m >= 3 && w.k >= 8192);
}

// Core dispatch. The caller holds h->mutex and has made h->device current.
int Dispatch(mnb_weights *h, const float *a_dev, std::int64_t m, int accuracy_level, int path,
             OutputView out, cudaStream_t stream) {
  if (accuracy_level != 0 && accuracy_level != 4) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits accuracy_level must be 0 or 4.");
  }
  if (m < 0) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits requires M >= 0.");
  }
  if (m == 0) {
    mnb::t_last_kernel = "none";
    return MNB_OK;
  }
  const WeightView &w = h->view;
  int chosen = path;
  if (chosen == MNB_PATH_AUTO) {
    if (accuracy_level == 4) {
      chosen = MNB_PATH_INT8_MMA; // falls through to the dp4a kernel when the shape does not fit
    } else if (m <= 16) {
      chosen = MNB_PATH_GEMV;
    } else {
      chosen = mnb::GemmTcgen05Supports(w, m) ? MNB_PATH_TCGEN05 : MNB_PATH_GEMV;
    }
  }
  const char *name = nullptr;
  switch (chosen) {
  case MNB_PATH_GEMV: {
    // decode default: the tensor-core kernels with the exact two-piece split. One column tile
    // holds 4 / 2 / 1 tokens for block_size >= 128 / 64 / 32; more tokens go to the kernel that
    // shares a pass over the weights between several column tiles.
    const int per_pass = w.block_size >= 128 ? 4 : (w.block_size == 64 ? 2 : 1);
    if (m == 1 && path == MNB_PATH_AUTO && mnb::DecodeResidentPreferred(w)) {
      // one token: the whole share of each SM is asked for at kernel start
      name = mnb::LaunchDecodeResident(w, a_dev, m, out, h->status_dev, stream, h->sm_count);
    }
    if (name == nullptr && m == 1 && path == MNB_PATH_AUTO) {
      // shapes the resident kernel does not take: every warp streams its own tile
      name = mnb::LaunchDecodeDirect(w, a_dev, m, out, stream, h->sm_count, true);
    }
    if (name == nullptr && m == 2 && path == MNB_PATH_AUTO && (w.k <= 2048 || (w.k >= 8192 && w.n >= 8192))) {
      // two tokens, long rows on a wide node or short rows: every warp streams its own tile (K = 14336,
      // N = 14336: 28.6 against 37.6 us on the integer-digit kernel below; K = 8192: 19.3 against 20.6;
      // K = 2048: 8.4 against 9.5 at N = 14336, 4.6 against 5.5 at N = 1024)
      name = mnb::LaunchDecodeDirect(w, a_dev, m, out, stream, h->sm_count, true);
    }
    if (name == nullptr && m <= kImmaAutoTokens && path == MNB_PATH_AUTO) {
      // one or two tokens, block_size >= 128: the integer-digit kernel (fewest instructions per code)
      name = mnb::LaunchGemvImma(w, a_dev, m, out, h->status_dev, stream, h->sm_count);
    }
    // Five and more tokens: all digit rows of a 2048-k slice in shared memory, one pass over the
    // weights (measured against the other paths, us per gate/up-sized node: block 32 M = 5 21.5 -> 20.2,
    // M = 8 34.1 -> 20.2, M = 16 47.1 -> 24.9; block 64 M = 8 32.8 -> 20.4; block 128 M = 5 20.3 -> 19.5,
    // M = 8 21.0 -> 19.5, M = 16 38.6 -> 25.7; four tokens stay on the fp16 kernel: 15.3 against 19.5).
    if (name == nullptr && m <= 16 && path == MNB_PATH_AUTO && DigitSlicesWanted(w, m)) {
      const std::size_t need = mnb::DigitSlicesScratchBytes(w, m);
      if (need != 0) {
        const int rc = Grow(&h->scratch_a, &h->scratch_a_bytes, need);
        if (rc != MNB_OK) {
          return rc;
        }
        name = mnb::LaunchDigitSlicesGroup(&w, &out, 1, a_dev, m, static_cast<unsigned char *>(h->scratch_a),
                                           h->status_dev, stream, h->sm_count);
        if (name == nullptr) {
          cudaGetLastError();
        }
      }
    }
    // Shapes the sliced kernel does not take: three digit rows per token through the sixteen-row
    // integer kernel in up to three passes, still fewer than one token per column tile on small blocks.
    if (name == nullptr && m <= 16 && path == MNB_PATH_AUTO &&
        ((w.block_size == 32 && m >= 5) || (w.block_size == 64 && m >= 9))) {
      const std::size_t need = mnb::DigitsInt8MmaScratchBytes(w, m);
      if (need != 0) {
        const int rc = Grow(&h->scratch_a, &h->scratch_a_bytes, need);
        if (rc != MNB_OK) {
          return rc;
        }
        name = mnb::LaunchDigitsInt8Mma(w, a_dev, m, static_cast<unsigned char *>(h->scratch_a), out,
                                        h->status_dev, stream, h->sm_count);
      }
    }
    if (name == nullptr && m <= 16 && path == MNB_PATH_AUTO) {
      if (m > per_pass) {
        name = mnb::LaunchGemvMmaMulti(w, a_dev, m, out, h->status_dev, stream, h->sm_count);
      }
      if (name == nullptr && m <= 4 * per_pass) {
        name = mnb::LaunchGemvMma(w, a_dev, m, out, h->status_dev, stream, h->sm_count);
      }
    }
    if (name == nullptr && m <= 16 && path == MNB_PATH_AUTO && w.bits == 8 &&
        (m >= 5 || (m >= 3 && ((w.n + 31) / 32 > h->sm_count || w.k > 4096)))) {
      // 8-bit weights, five tokens and more (three and more on nodes wider than one 32-column CTA per SM and
      // on rows of more than 4096 k, where the lane-per-column kernel takes 52 us at K = 14336, N = 4096, M = 4):
      // digit columns on integer tensor cores, one pass over the weights and one duration for one to eight
      // tokens (us per call against the CUDA-core kernels below, K = 4096: N = 16032 block 32 45 against 29 at
      // M = 2, 53 at M = 3, 54 at M = 4 and 95 at M = 8; N = 4096 block 64 21 against 17 at M = 3, 4 and
      // 23 / 41 at M = 8 / 16)
      const std::size_t need = mnb::GemvU8MmaScratchBytes(w, m);
      if (need != 0) {
        const int rc = Grow(&h->scratch_a, &h->scratch_a_bytes, need);
        if (rc != MNB_OK) {
          return rc;
        }
        name = mnb::LaunchGemvU8Mma(w, a_dev, m, static_cast<unsigned char *>(h->scratch_a), out, stream, h->sm_count);
        if (name == nullptr) {
          cudaGetLastError();
        }
      }
    }
    if (name == nullptr && m <= 16 && path == MNB_PATH_AUTO && w.bits == 8 &&
        (m >= 8 || (m >= 3 && (w.n + 31) / 32 <= h->sm_count))) {
      // 8-bit weights: the staged kernel below takes two tokens per pass over the weights, the
      // lane-per-column kernel eight. Measured, us per call, staged against lane-per-column:
      // K = 4096, N = 14336 M = 4 / 8 / 16: 51.8 / 97.1 / 189 against 56.0 / 81.3 / 148;
      // K = 8192, N = 4096: M = 3 / 8 / 16 42.7 / 83.6 / 161 against 31.4 / 45.5 / 78.5 (a node of at
      // most one 32-column CTA per SM runs sixteen warps along K).
      name = mnb::LaunchGemvWords(w, a_dev, m, out, stream, h->sm_count);
    }
    if (name == nullptr && m <= 16) {
      name = mnb::LaunchGemvStream(w, a_dev, m, out, h->status_dev, stream, h->sm_count);
    }
    if (name == nullptr && m <= 16 && path == MNB_PATH_AUTO) {
      // shapes the CUDA-core kernel cannot stage (very long K with several tokens): many passes of
      // the tensor-core kernel still beat the generic one by a wide margin
      name = mnb::LaunchGemvMma(w, a_dev, m, out, h->status_dev, stream, h->sm_count);
    }
    if (name == nullptr && m <= 16 && path == MNB_PATH_AUTO && w.bits == 4) {
      // nothing above took the shape: the one-pass digit kernel, whatever the token count, before the
      // generic kernel (two to three orders of magnitude slower)
      const std::size_t need = mnb::DigitSlicesScratchBytes(w, m);
      if (need != 0) {
        const int rc = Grow(&h->scratch_a, &h->scratch_a_bytes, need);
        if (rc != MNB_OK) {
          return rc;
        }
        name = mnb::LaunchDigitSlicesGroup(&w, &out, 1, a_dev, m, static_cast<unsigned char *>(h->scratch_a),
                                           h->status_dev, stream, h->sm_count);
        if (name == nullptr) {
          cudaGetLastError();
        }
      }
    }
    if (name == nullptr && m >= 2 && m <= 16 && path == MNB_PATH_AUTO && w.bits == 8) {
      // 8-bit rows too long for the staged kernel, two to four tokens: the tensor-core kernel before the
      // word-wise ones (K = 14336, N = 4096, M = 2: 33 against 42 us)
      const std::size_t need = mnb::GemvU8MmaScratchBytes(w, m);
      if (need != 0) {
        const int rc = Grow(&h->scratch_a, &h->scratch_a_bytes, need);
        if (rc != MNB_OK) {
          return rc;
        }
        name = mnb::LaunchGemvU8Mma(w, a_dev, m, static_cast<unsigned char *>(h->scratch_a), out, stream, h->sm_count);
        if (name == nullptr) {
          cudaGetLastError();
        }
      }
    }
    if (name == nullptr) {
      name = mnb::LaunchGemvGeneric(w, a_dev, m, out, stream, h->sm_count);
    }
    break;
  }
  case MNB_PATH_GEMV_MMA: {
    name = mnb::LaunchGemvMma(w, a_dev, m, out, h->status_dev, stream, h->sm_count);
    if (name == nullptr) {
      return Fail(MNB_ERR_UNSUPPORTED, "MatMulNBits: shape not supported by the MMA decode kernel.");
    }
    break;
  }
  case MNB_PATH_GEMV_IMMA: {
    name = mnb::LaunchGemvImma(w, a_dev, m, out, h->status_dev, stream, h->sm_count);
    if (name == nullptr) {
      return Fail(MNB_ERR_UNSUPPORTED,
                  "MatMulNBits: the integer-digit decode kernel takes 4-bit weights with block_size 128 ... "
                  "1024 and M <= 16.");
    }
    break;
  }
  case MNB_PATH_GEMV_DIRECT: {
    name = m <= 2 ? mnb::LaunchDecodeDirect(w, a_dev, m, out, stream, h->sm_count, true) : nullptr;
    if (name == nullptr) {
      return Fail(MNB_ERR_UNSUPPORTED,
                  "MatMulNBits: the direct-stream decode kernel takes 4-bit weights with block_size 128, a "
                  "number of blocks per row that is a multiple of 4, 16-byte aligned operands and M <= 2.");
    }
    break;
  }
  case MNB_PATH_GEMV_RESIDENT: {
    name = mnb::LaunchDecodeResident(w, a_dev, m, out, h->status_dev, stream, h->sm_count);
    if (name == nullptr) {
      return Fail(MNB_ERR_UNSUPPORTED,
                  "MatMulNBits: the resident decode kernel takes one token, 4-bit weights with block_size 128, K a "
                  "multiple of 1024 (2048 with zero points) and 16-byte aligned operands.");
    }
    break;
  }
  case MNB_PATH_GEMV_DIGITS: {
    const std::size_t sliced = m <= 16 ? mnb::DigitSlicesScratchBytes(w, m) : 0;
    if (sliced != 0) {
      const int rc = Grow(&h->scratch_a, &h->scratch_a_bytes, sliced);
      if (rc != MNB_OK) {
        return rc;
      }
      name = mnb::LaunchDigitSlicesGroup(&w, &out, 1, a_dev, m, static_cast<unsigned char *>(h->scratch_a),
                                         h->status_dev, stream, h->sm_count);
      if (name != nullptr) {
        break;
      }
      cudaGetLastError();
    }
    const std::size_t need = m <= 16 ? mnb::DigitsInt8MmaScratchBytes(w, m) : 0;
    if (need != 0) {
      const int rc = Grow(&h->scratch_a, &h->scratch_a_bytes, need);
      if (rc != MNB_OK) {
        return rc;
      }
      name = mnb::LaunchDigitsInt8Mma(w, a_dev, m, static_cast<unsigned char *>(h->scratch_a), out, h->status_dev,
                                      stream, h->sm_count);
    }
    if (name == nullptr) {
      return Fail(MNB_ERR_UNSUPPORTED,
                  "MatMulNBits: the digit-row decode path needs bits=4, 32 <= block_size <= 1024, packed rows "
                  "that are a multiple of 128 bytes and M <= 16.");
    }
    break;
  }
  case MNB_PATH_GEMV_MMA_MULTI: {
    name = mnb::LaunchGemvMmaMulti(w, a_dev, m, out, h->status_dev, stream, h->sm_count);
    if (name == nullptr) {
      return Fail(MNB_ERR_UNSUPPORTED,
                  "MatMulNBits: the multi-tile MMA decode kernel needs more tokens than one column tile "
                  "holds (4 / 2 / 1 for block_size >= 128 / 64 / 32), M <= 16 and a supported shape.");
    }
    break;
  }
  case MNB_PATH_TCGEN05:
  case MNB_PATH_TCGEN05_WIDE: {
    if (!mnb::GemmTcgen05Supports(w, m)) {
      return Fail(MNB_ERR_UNSUPPORTED,
                  "MatMulNBits: the tcgen05 path needs bits 4 or 8, block_size>=32, K%64==0.");
    }
    const int rc = Grow(&h->scratch_a, &h->scratch_a_bytes, mnb::GemmTcgen05ScratchBytes(w, m, h->sm_count));
    if (rc != MNB_OK) {
      return rc;
    }
    name = mnb::LaunchGemmTcgen05(w, a_dev, m, static_cast<std::uint16_t *>(h->scratch_a), out,
                                  h->status_dev, stream, h->sm_count,
                                  path == MNB_PATH_AUTO ? mnb::kGemmTileAuto
                                                        : (path == MNB_PATH_TCGEN05_WIDE ? mnb::kGemmTilePairs : mnb::kGemmTileRows128));
    break;
  }
  case MNB_PATH_INT8_MMA: {
    const std::size_t need = mnb::Int8MmaScratchBytes(w, m);
    if (need != 0) {
      const int rc = Grow(&h->scratch_a, &h->scratch_a_bytes, need);
      if (rc != MNB_OK) {
        return rc;
      }
      name = mnb::LaunchInt8Mma(w, a_dev, m, static_cast<unsigned char *>(h->scratch_a), out, h->status_dev,
                                stream, h->sm_count);
    }
    if (name != nullptr) {
      break;
    }
    if (path == MNB_PATH_INT8_MMA) {
      return Fail(MNB_ERR_UNSUPPORTED,
                  "MatMulNBits: the integer-MMA path needs bits=4, 32 <= block_size <= 1024 and packed "
                  "rows that are a multiple of 128 bytes.");
    }
  }
    [[fallthrough]];
  case MNB_PATH_INT8: {
    const std::size_t aq_bytes = static_cast<std::size_t>(m) * w.n_blocks * w.block_size;
    int rc = Grow(&h->scratch_a, &h->scratch_a_bytes, aq_bytes);
    if (rc != MNB_OK) {
      return rc;
    }
    // activation scales, and behind them room for the per-block sums of the 8-bit tensor-core kernel
    const std::size_t scale_count = static_cast<std::size_t>(m) * w.n_blocks;
    rc = Grow(&h->scratch_s, &h->scratch_s_bytes, scale_count * (sizeof(float) + sizeof(int)));
    if (rc != MNB_OK) {
      return rc;
    }
    name = mnb::LaunchQuantizeAPadded(a_dev, m, w.k, w.block_size,
                                      static_cast<std::int8_t *>(h->scratch_a),
                                      static_cast<float *>(h->scratch_s), stream);
    if (name != nullptr && path == MNB_PATH_AUTO && mnb::GemvU8MmaSupports(w, m)) {
      // 8-bit weights, up to sixteen tokens: the quantized activations as columns of an integer MMA
      const char *mma = mnb::LaunchGemvU8Int8Mma(w, static_cast<const std::int8_t *>(h->scratch_a),
                                                 static_cast<const float *>(h->scratch_s), m,
                                                 reinterpret_cast<int *>(static_cast<float *>(h->scratch_s) + scale_count), out,
                                                 stream, h->sm_count);
      if (mma != nullptr) {
        name = mma;
        break;
      }
      cudaGetLastError();
    }
    if (name != nullptr) {
      name = mnb::LaunchInt8Matmul(w, static_cast<const std::int8_t *>(h->scratch_a),
                                   static_cast<const float *>(h->scratch_s), m, out, stream,
                                   h->sm_count);
    }
    if (name == nullptr) {
      return Fail(MNB_ERR_UNSUPPORTED,
                  "MatMulNBits: accuracy_level 4 needs packed rows and a weight base aligned to eight codes "
                  "(4 bytes for 4-bit, 8 bytes for 8-bit weights).");
    }
    break;
  }
  default:
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits: unknown path selector.");
  }
  if (name == nullptr) {
    const cudaError_t err = cudaGetLastError();
    return Fail(MNB_ERR_CUDA, std::string("matmulnbits_b200: kernel launch failed: ") +
                                  cudaGetErrorString(err));
  }
  mnb::t_last_kernel = name;
  return MNB_OK;
}

// Device memory of another GPU would be read through an address this GPU cannot reach, and
// plain host memory through no address at all (a fault, not an error code): checks where A and Y
// live, once per pointer pair of the handle. Allocates nothing. The caller holds h->mutex.
int CheckDeviceOperands(mnb_weights *h, const void *a_dev, const void *y_dev) {
  if (a_dev == h->checked_a && y_dev == h->checked_y) {
    return MNB_OK;
  }
  for (const void *ptr : {a_dev, y_dev}) {
    cudaPointerAttributes attributes{};
    const cudaError_t query = cudaPointerGetAttributes(&attributes, ptr);
    if (query != cudaSuccess) {
      cudaGetLastError();
      continue; // not known to the runtime: leave the decision to the launch
    }
    if (attributes.type == cudaMemoryTypeDevice && attributes.device != h->device) {
      char text[160];
      std::snprintf(text, sizeof(text),
                    "MatMulNBits: A and Y must be memory of GPU %d, where the weights are (got memory of GPU %d).",
                    h->device, attributes.device);
      return Fail(MNB_ERR_INVALID_ARGUMENT, text);
    }
    if (attributes.type == cudaMemoryTypeUnregistered) {
      return Fail(MNB_ERR_INVALID_ARGUMENT,
                  "MatMulNBits: the device-pointer entry points take device memory; use mnb_matmul_host for "
                  "host buffers.");
    }
  }
  h->checked_a = a_dev;
  h->checked_y = y_dev;
  return MNB_OK;
}

} // namespace

extern "C" {

const char *mnb_last_error(void) { return mnb::t_last_error.c_str(); }

const char *mnb_version(void) { return "matmulnbits_b200 0.1.0 sm_100a"; }

int mnb_device_count(int *count) {
  if (count == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_device_count: null output.");
  }
  int n = 0;
  const cudaError_t err = cudaGetDeviceCount(&n);
  if (err != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  *count = n;
  return MNB_OK;
}

int64_t mnb_algorithmic_bytes(int64_t m, int64_t n, int64_t k, int bits, int block_size,
                              int has_zero_points, int has_bias) {
  const int64_t n_blocks = (k + block_size - 1) / block_size;
  int64_t bytes = n * n_blocks * (static_cast<int64_t>(block_size) * bits / 8);
  bytes += 4 * n * n_blocks;
  if (has_zero_points) {
    bytes += n * ((n_blocks * bits + 7) / 8);
  }
  if (has_bias) {
    bytes += 4 * n;
  }
  bytes += 4 * m * k + 4 * m * n;
  return bytes;
}

static int CreateImpl(int device, const uint8_t *b, const float *scales, const uint8_t *zero_points,
                      const float *bias, int64_t n, int64_t k, int bits, int block_size, bool copy,
                      mnb_weights **out) {
  if (out == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_weights_create: null output handle.");
  }
  *out = nullptr;
  std::string why;
  if (!ValidGeometry(n, k, bits, block_size, &why)) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, why);
  }
  if (b == nullptr || scales == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits requires B and scales.");
  }
  int count = 0;
  mnb_device_count(&count);
  if (count <= 0) {
    return Fail(MNB_ERR_CUDA, "matmulnbits_b200: no CUDA device is visible; there is no CPU path.");
  }
  if (device < 0 || device >= count) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "matmulnbits_b200: device index out of range.");
  }
  mnb_weights *h = new (std::nothrow) mnb_weights();
  if (h == nullptr) {
    return Fail(MNB_ERR_CUDA, "matmulnbits_b200: out of host memory.");
  }
  h->device = device;
  FillView(&h->view, n, k, bits, block_size);
  int rc = SetupCommon(h);
  if (rc != MNB_OK) {
    mnb_weights_destroy(h);
    return rc;
  }
  if (!copy) {
    h->view.b = b;
    h->view.scales = scales;
    h->view.zp = zero_points;
    h->view.bias = bias;
    rc = PrepareMeta(h);
    if (rc != MNB_OK) {
      mnb_weights_destroy(h);
      return rc;
    }
    *out = h;
    return MNB_OK;
  }
  h->owns = true;
  const std::size_t sizes[4] = {
      static_cast<std::size_t>(n) * h->view.row_bytes,
      static_cast<std::size_t>(n) * h->view.n_blocks * sizeof(float),
      zero_points != nullptr ? static_cast<std::size_t>(n) * h->view.zp_row_bytes : 0,
      bias != nullptr ? static_cast<std::size_t>(n) * sizeof(float) : 0};
  const void *sources[4] = {b, scales, zero_points, bias};
  for (int i = 0; i < 4; ++i) {
    if (sizes[i] == 0) {
      continue;
    }
    cudaError_t err = cudaMalloc(&h->owned[i], sizes[i]);
    if (err == cudaSuccess) {
      err = cudaMemcpy(h->owned[i], sources[i], sizes[i], cudaMemcpyHostToDevice);
    }
    if (err != cudaSuccess) {
      rc = FailCuda("weight upload", err);
      mnb_weights_destroy(h);
      return rc;
    }
  }
  h->view.b = static_cast<const std::uint8_t *>(h->owned[0]);
  h->view.scales = static_cast<const float *>(h->owned[1]);
  h->view.zp = static_cast<const std::uint8_t *>(h->owned[2]);
  h->view.bias = static_cast<const float *>(h->owned[3]);
  rc = PrepareMeta(h);
  if (rc != MNB_OK) {
    mnb_weights_destroy(h);
    return rc;
  }
  *out = h;
  return MNB_OK;
}

int mnb_weights_create(int device, const uint8_t *b, const float *scales,
                       const uint8_t *zero_points, const float *bias, int64_t n, int64_t k,
                       int bits, int block_size, mnb_weights **out) {
  return CreateImpl(device, b, scales, zero_points, bias, n, k, bits, block_size, true, out);
}

int mnb_weights_wrap_device(int device, const uint8_t *b, const float *scales,
                            const uint8_t *zero_points, const float *bias, int64_t n, int64_t k,
                            int bits, int block_size, mnb_weights **out) {
  return CreateImpl(device, b, scales, zero_points, bias, n, k, bits, block_size, false, out);
}

int mnb_weights_destroy(mnb_weights *h) {
  if (h == nullptr) {
    return MNB_OK;
  }
  cudaSetDevice(h->device);
  mnb::ForgetDecodeResidentPlans(h->view);
  if (h->stream != nullptr) {
    cudaStreamSynchronize(h->stream);
    cudaStreamDestroy(h->stream);
  }
  if (h->owns) {
    for (void *ptr : h->owned) {
      if (ptr != nullptr) {
        cudaFree(ptr);
      }
    }
  }
  for (void *ptr : {static_cast<void *>(h->arrivals_dev), h->meta_dev, h->zp16_dev, h->scratch_a, h->scratch_s,
                    static_cast<void *>(h->a_dev), static_cast<void *>(h->y_dev)}) {
    if (ptr != nullptr) {
      cudaFree(ptr);
    }
  }
  if (h->status_host != nullptr) {
    cudaFreeHost(h->status_host);
  }
  delete h;
  return MNB_OK;
}

int mnb_matmul_device_strided(mnb_weights *h, const float *a_dev, int64_t m, int accuracy_level,
                              int path, float *y_dev, int64_t ld_y, int64_t col_offset,
                              void *stream) {
  if (h == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits: null weights handle.");
  }
  if (m > 0 && (a_dev == nullptr || y_dev == nullptr)) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits: null A or Y.");
  }
  if (ld_y < h->view.n || col_offset < 0 || col_offset + h->view.n > ld_y) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits: output window does not fit its row.");
  }
  std::lock_guard<std::mutex> guard(h->mutex);
  const cudaError_t err = cudaSetDevice(h->device);
  if (err != cudaSuccess) {
    return FailCuda("cudaSetDevice", err);
  }
  if (m > 0) {
    const int rc = CheckDeviceOperands(h, a_dev, y_dev);
    if (rc != MNB_OK) {
      return rc;
    }
  }
  OutputView out{y_dev, ld_y, col_offset};
  return Dispatch(h, a_dev, m, accuracy_level, path, out, static_cast<cudaStream_t>(stream));
}

static_assert(MNB_MAX_GROUPED_NODES == mnb::kMaxGroupedNodes, "header and kernels agree on the group size");

int mnb_matmul_device_group(mnb_weights *const *handles, int count, const float *a_dev, int64_t m,
                            int accuracy_level, float *const *y_dev, void *stream) {
  if (handles == nullptr || y_dev == nullptr || count < 1 || count > MNB_MAX_GROUPED_NODES) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_matmul_device_group: takes 1 to 3 nodes.");
  }
  if (accuracy_level != 0 && accuracy_level != 4) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits accuracy_level must be 0 or 4.");
  }
  if (m < 0) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits requires M >= 0.");
  }
  for (int i = 0; i < count; ++i) {
    if (handles[i] == nullptr) {
      return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits: null weights handle.");
    }
    if (m > 0 && (a_dev == nullptr || y_dev[i] == nullptr)) {
      return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits: null A or Y.");
    }
    if (handles[i]->device != handles[0]->device || handles[i]->view.k != handles[0]->view.k) {
      return Fail(MNB_ERR_INVALID_ARGUMENT,
                  "mnb_matmul_device_group: the nodes of a group take the same A: same K, same GPU.");
    }
    for (int j = 0; j < i; ++j) {
      if (handles[j] == handles[i] || y_dev[j] == y_dev[i]) {
        return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_matmul_device_group: a node or an output is named twice.");
      }
    }
  }
  // every node's lock, in address order so that two groups over the same nodes cannot block each other
  mnb_weights *ordered[MNB_MAX_GROUPED_NODES];
  for (int i = 0; i < count; ++i) {
    ordered[i] = handles[i];
  }
  std::sort(ordered, ordered + count);
  std::unique_lock<std::mutex> locks[MNB_MAX_GROUPED_NODES];
  for (int i = 0; i < count; ++i) {
    locks[i] = std::unique_lock<std::mutex>(ordered[i]->mutex);
  }
  mnb_weights *first = handles[0];
  const cudaError_t err = cudaSetDevice(first->device);
  if (err != cudaSuccess) {
    return FailCuda("cudaSetDevice", err);
  }
  if (m == 0) {
    mnb::t_last_kernel = "none";
    return MNB_OK;
  }
  WeightView nodes[MNB_MAX_GROUPED_NODES];
  OutputView outs[MNB_MAX_GROUPED_NODES];
  for (int i = 0; i < count; ++i) {
    const int rc = CheckDeviceOperands(handles[i], a_dev, y_dev[i]);
    if (rc != MNB_OK) {
      return rc;
    }
    nodes[i] = handles[i]->view;
    outs[i] = OutputView{y_dev[i], handles[i]->view.n, 0};
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const char *name = nullptr;
  // Bounded waits of a grouped launch report through the first node's status word.
  if (accuracy_level == 0 && m == 1 && mnb::DecodeResidentGroupPreferred(nodes, count)) {
    // one launch: the nodes' tiles form one sequence behind activations staged once
    name = mnb::LaunchDecodeResidentGroup(nodes, outs, count, a_dev, m, first->status_dev, s, first->sm_count);
  } else if (accuracy_level == 4 && count > 1) {
    // activations quantized once, then one integer-MMA launch per node
    std::size_t need = 0;
    for (int i = 0; i < count; ++i) {
      const std::size_t bytes = mnb::Int8MmaScratchBytes(nodes[i], m);
      need = bytes == 0 ? 0 : (bytes > need ? bytes : need);
      if (bytes == 0) {
        break;
      }
    }
    if (need != 0) {
      const int rc = Grow(&first->scratch_a, &first->scratch_a_bytes, need);
      if (rc != MNB_OK) {
        return rc;
      }
      name = mnb::LaunchInt8MmaGroup(nodes, outs, count, a_dev, m, static_cast<unsigned char *>(first->scratch_a),
                                     first->status_dev, s, first->sm_count);
    }
  } else if (accuracy_level == 0 && count > 1 && m <= 16 && DigitSlicesWanted(nodes[0], m)) {
    // the digit rows of all K slices made once, one product launch for all nodes, then a sum per node
    const std::size_t need = mnb::DigitSlicesGroupScratchBytes(nodes, count, m);
    if (need != 0) {
      const int rc = Grow(&first->scratch_a, &first->scratch_a_bytes, need);
      if (rc != MNB_OK) {
        return rc;
      }
      name = mnb::LaunchDigitSlicesGroup(nodes, outs, count, a_dev, m, static_cast<unsigned char *>(first->scratch_a),
                                         first->status_dev, s, first->sm_count);
    }
  } else if (accuracy_level == 0 && count > 1 && m <= 16 &&
             ((nodes[0].block_size == 32 && m >= 5) || (nodes[0].block_size == 64 && m >= 9))) {
    // digit rows made once, then the three-pass integer-MMA product and its combine per node
    std::size_t need = 0;
    for (int i = 0; i < count; ++i) {
      const std::size_t bytes = mnb::DigitsInt8MmaScratchBytes(nodes[i], m);
      need = bytes == 0 ? 0 : (bytes > need ? bytes : need);
      if (bytes == 0) {
        break;
      }
    }
    if (need != 0) {
      const int rc = Grow(&first->scratch_a, &first->scratch_a_bytes, need);
      if (rc != MNB_OK) {
        return rc;
      }
      name = mnb::LaunchDigitsInt8MmaGroup(nodes, outs, count, a_dev, m,
                                           static_cast<unsigned char *>(first->scratch_a), first->status_dev, s,
                                           first->sm_count);
    }
  }
  if (name != nullptr) {
    mnb::t_last_kernel = name;
    return MNB_OK;
  }
  cudaGetLastError();
  // no shared form for this group: node by node, as separate calls would run
  for (int i = 0; i < count; ++i) {
    const int rc = Dispatch(handles[i], a_dev, m, accuracy_level, MNB_PATH_AUTO, outs[i], s);
    if (rc != MNB_OK) {
      return rc;
    }
  }
  return MNB_OK;
}

int mnb_peer_buffer_create(int device, size_t bytes, void **dev_ptr, unsigned char *handle_out) {
  static_assert(sizeof(cudaIpcMemHandle_t) == MNB_IPC_HANDLE_BYTES, "handle size");
  if (dev_ptr == nullptr || handle_out == nullptr || bytes == 0) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_peer_buffer_create: null argument or zero size.");
  }
  cudaError_t err = cudaSetDevice(device);
  if (err != cudaSuccess) {
    return FailCuda("cudaSetDevice", err);
  }
  void *ptr = nullptr;
  err = cudaMalloc(&ptr, bytes);
  if (err != cudaSuccess) {
    return FailCuda("cudaMalloc(peer buffer)", err);
  }
  err = cudaMemset(ptr, 0, bytes);
  cudaIpcMemHandle_t handle;
  if (err == cudaSuccess) {
    err = cudaIpcGetMemHandle(&handle, ptr);
  }
  if (err != cudaSuccess) {
    cudaFree(ptr);
    return FailCuda("cudaIpcGetMemHandle", err);
  }
  std::memcpy(handle_out, &handle, sizeof(handle));
  *dev_ptr = ptr;
  return MNB_OK;
}

int mnb_peer_buffer_open(int device, const unsigned char *handle_bytes, void **peer_ptr) {
  if (handle_bytes == nullptr || peer_ptr == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_peer_buffer_open: null argument.");
  }
  cudaError_t err = cudaSetDevice(device);
  if (err != cudaSuccess) {
    return FailCuda("cudaSetDevice", err);
  }
  cudaIpcMemHandle_t handle;
  std::memcpy(&handle, handle_bytes, sizeof(handle));
  err = cudaIpcOpenMemHandle(peer_ptr, handle, cudaIpcMemLazyEnablePeerAccess);
  if (err != cudaSuccess) {
    return FailCuda("cudaIpcOpenMemHandle", err);
  }
  // Copies into the mapping work as soon as it exists, loads and stores from kernels only once
  // peer access to the owning device is enabled for this context: do it here, explicitly.
  cudaPointerAttributes attributes{};
  err = cudaPointerGetAttributes(&attributes, *peer_ptr);
  if (err == cudaSuccess && attributes.device >= 0 && attributes.device != device) {
    int can = 0;
    err = cudaDeviceCanAccessPeer(&can, device, attributes.device);
    if (err == cudaSuccess && can == 0) {
      cudaIpcCloseMemHandle(*peer_ptr);
      *peer_ptr = nullptr;
      return Fail(MNB_ERR_UNSUPPORTED, "mnb_peer_buffer_open: the two GPUs cannot address each other's memory.");
    }
    if (err == cudaSuccess) {
      err = cudaDeviceEnablePeerAccess(attributes.device, 0);
      if (err == cudaErrorPeerAccessAlreadyEnabled) {
        err = cudaSuccess;
      }
    }
  }
  cudaGetLastError(); // drop the benign "already enabled"
  if (err != cudaSuccess) {
    cudaIpcCloseMemHandle(*peer_ptr);
    *peer_ptr = nullptr;
    return FailCuda("enabling peer access", err);
  }
  return MNB_OK;
}

int mnb_peer_buffer_close(int device, void *peer_ptr) {
  if (peer_ptr == nullptr) {
    return MNB_OK;
  }
  cudaSetDevice(device);
  const cudaError_t err = cudaIpcCloseMemHandle(peer_ptr);
  return err == cudaSuccess ? MNB_OK : FailCuda("cudaIpcCloseMemHandle", err);
}

int mnb_peer_buffer_destroy(int device, void *dev_ptr) {
  if (dev_ptr == nullptr) {
    return MNB_OK;
  }
  cudaSetDevice(device);
  const cudaError_t err = cudaFree(dev_ptr);
  return err == cudaSuccess ? MNB_OK : FailCuda("cudaFree(peer buffer)", err);
}

namespace {

int LaunchGatherWait(mnb_weights *h, int *const *flags_local, const int *epochs, int count, int ranks,
                     cudaStream_t stream) {
  GatherWaitList list{};
  list.count = count;
  list.ranks = ranks;
  for (int i = 0; i < count; ++i) {
    list.flags[i] = flags_local[i];
    list.epoch[i] = epochs != nullptr ? epochs[i] : 0;
  }
  cudaGetLastError(); // drop any stale, non-sticky error so that the check below reads this launch
  nbits_gather_wait_kernel<<<1, 32 * count, 0, stream>>>(list, h->status_dev);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    return FailCuda("launch of the gather wait kernel", err);
  }
  mnb::CountLaunch();
  return MNB_OK;
}

} // namespace

int mnb_matmul_device_gather_ex(mnb_weights *h, const float *a_dev, int64_t m, int accuracy_level,
                                float *const *y_ranks, int *const *flags_ranks, int ranks, int rank, int64_t ld_y,
                                int64_t col_offset, int epoch, int wait, void *stream_ptr) {
  if (h == nullptr || a_dev == nullptr || y_ranks == nullptr || flags_ranks == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_matmul_device_gather: null argument.");
  }
  if (ranks < 1 || ranks > MNB_MAX_GATHER_RANKS || rank < 0 || rank >= ranks) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_matmul_device_gather: 1 <= ranks <= 8 and 0 <= rank < ranks.");
  }
  if (m < 1) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_matmul_device_gather: M >= 1.");
  }
  if (accuracy_level != 0 && accuracy_level != 4) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits accuracy_level must be 0 or 4.");
  }
  if (ld_y < h->view.n || col_offset < 0 || col_offset + h->view.n > ld_y) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits: output window does not fit its row.");
  }
  for (int r = 0; r < ranks; ++r) {
    if (y_ranks[r] == nullptr || flags_ranks[r] == nullptr) {
      return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_matmul_device_gather: null buffer in the rank tables.");
    }
  }
  std::lock_guard<std::mutex> guard(h->mutex);
  const cudaError_t err = cudaSetDevice(h->device);
  if (err != cudaSuccess) {
    return FailCuda("cudaSetDevice", err);
  }
  // A and the local result must live on the GPU that holds the weights: a handle created on
  // another device (the default device of a second rank, say) would otherwise read them through
  // an address that GPU cannot reach.
  for (const void *ptr : {static_cast<const void *>(a_dev), static_cast<const void *>(y_ranks[rank])}) {
    cudaPointerAttributes attributes{};
    if (cudaPointerGetAttributes(&attributes, ptr) != cudaSuccess || attributes.type != cudaMemoryTypeDevice ||
        attributes.device != h->device) {
      cudaGetLastError();
      return Fail(MNB_ERR_INVALID_ARGUMENT,
                  "mnb_matmul_device_gather: A and the local result buffer must be device memory of the GPU "
                  "the weights were created on.");
    }
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  OutputView out{y_ranks[rank], ld_y, col_offset};
  mnb::GatherTail tail{};
  tail.ranks = ranks;
  tail.rank = rank;
  tail.epoch = epoch;
  tail.wait = 0;
  tail.arrivals = h->arrivals_dev;
  for (int r = 0; r < ranks; ++r) {
    tail.flags[r] = flags_ranks[r];
    if (r != rank) {
      tail.peers[tail.n_peers++] = y_ranks[r];
    }
  }
  const WeightView &w = h->view;
  const char *name = nullptr;
  // (token counts that AUTO sends to the one-pass digit kernel take the general path below: that
  // kernel plus the push is faster than the decode kernels with their own push, 100 against 157 us
  // per lm-head half at M = 8)
  if (accuracy_level == 0 && m <= 16 && !(DigitSlicesWanted(w, m) && mnb::DigitSlicesScratchBytes(w, m) != 0)) {
    mnb::GatherTail fused_tail = tail;
    fused_tail.wait = wait != 0 ? 1 : 0;
    // The tensor-core decode kernels push each CTA's rows to the peers as the CTA finishes, and the
    // last CTA to finish publishes the flags: one launch per node, no pass over the result.
    const int per_pass = w.block_size >= 128 ? 4 : (w.block_size == 64 ? 2 : 1);
    if (m == 1 && mnb::DecodeResidentSupports(w, m) && mnb::DecodeResidentPreferred(w)) {
      // one token: the kernel that asks for each SM's whole share of the weights at its start
      name = mnb::LaunchDecodeResident(w, a_dev, m, out, h->status_dev, stream, h->sm_count, &fused_tail);
      if (name == nullptr) {
        cudaGetLastError();
      }
    }
    if (name == nullptr && m > per_pass) {
      name = mnb::LaunchGemvMmaMulti(w, a_dev, m, out, h->status_dev, stream, h->sm_count, &fused_tail);
    }
    if (name == nullptr) {
      name = mnb::LaunchGemvMma(w, a_dev, m, out, h->status_dev, stream, h->sm_count, &fused_tail);
    }
  }
  if (name == nullptr) {
    // Any other shape (8-bit weights, prefill sizes, accuracy_level 4): the product goes to the local
    // window through the ordinary dispatch, then one kernel copies the window to the peers and
    // publishes.
    cudaGetLastError();
    OutputView local{y_ranks[rank], ld_y, col_offset};
    const int rc = Dispatch(h, a_dev, m, accuracy_level, MNB_PATH_AUTO, local, stream);
    if (rc != MNB_OK) {
      return rc;
    }
    name = mnb::t_last_kernel;
    bool vector = (w.n % 4) == 0 && (ld_y % 4) == 0 && (col_offset % 4) == 0;
    for (int r = 0; r < ranks; ++r) {
      vector = vector && (reinterpret_cast<std::uintptr_t>(y_ranks[r]) & 15u) == 0;
    }
    const std::int64_t items = vector ? m * (w.n / 4) : m * w.n;
    std::int64_t blocks = (items + 255) / 256;
    const std::int64_t most = 2 * static_cast<std::int64_t>(h->sm_count > 0 ? h->sm_count : 148);
    blocks = blocks > most ? most : (blocks < 1 ? 1 : blocks);
    tail.wait = wait != 0 ? 1 : 0;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
    config.blockDim = dim3(256, 1, 1);
    config.dynamicSmemBytes = 0;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    const cudaError_t launch_err = cudaLaunchKernelEx(&config, nbits_gather_push_kernel, out, static_cast<std::int64_t>(m),
                                                      static_cast<std::int64_t>(w.n), vector ? 1 : 0, tail, h->status_dev);
    if (launch_err != cudaSuccess) {
      return FailCuda("launch of the gather push kernel", launch_err);
    }
    mnb::CountLaunch();
  }
  mnb::t_last_kernel = name;
  return MNB_OK;
}

int mnb_matmul_device_gather(mnb_weights *h, const float *a_dev, int64_t m, float *const *y_ranks,
                             int *const *flags_ranks, int ranks, int rank, int64_t ld_y, int64_t col_offset,
                             int epoch, void *stream_ptr) {
  return mnb_matmul_device_gather_ex(h, a_dev, m, 0, y_ranks, flags_ranks, ranks, rank, ld_y, col_offset, epoch, 1,
                                     stream_ptr);
}

int mnb_gather_wait(mnb_weights *h, int *const *flags_local, const int *epochs, int count, int ranks,
                    void *stream_ptr) {
  if (h == nullptr || flags_local == nullptr || count < 1 || count > MNB_MAX_GATHER_WAITS || ranks < 1 ||
      ranks > MNB_MAX_GATHER_RANKS) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_gather_wait: 1 to 8 flag arrays of 1 to 8 ranks.");
  }
  for (int i = 0; i < count; ++i) {
    if (flags_local[i] == nullptr) {
      return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_gather_wait: null flag array.");
    }
  }
  std::lock_guard<std::mutex> guard(h->mutex);
  const cudaError_t err = cudaSetDevice(h->device);
  if (err != cudaSuccess) {
    return FailCuda("cudaSetDevice", err);
  }
  return LaunchGatherWait(h, flags_local, epochs, count, ranks, static_cast<cudaStream_t>(stream_ptr));
}

int mnb_matmul_device(mnb_weights *h, const float *a_dev, int64_t m, int accuracy_level, int path,
                      float *y_dev, void *stream) {
  if (h == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits: null weights handle.");
  }
  return mnb_matmul_device_strided(h, a_dev, m, accuracy_level, path, y_dev, h->view.n, 0, stream);
}

int mnb_matmul_host(mnb_weights *h, const float *a_host, int64_t m, int accuracy_level, int path,
                    float *y_host) {
  if (h == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits: null weights handle.");
  }
  if (m < 0) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits requires M >= 0.");
  }
  if (m == 0) {
    return MNB_OK;
  }
  if (a_host == nullptr || y_host == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "MatMulNBits: null A or Y.");
  }
  std::lock_guard<std::mutex> guard(h->mutex);
  cudaError_t err = cudaSetDevice(h->device);
  if (err != cudaSuccess) {
    return FailCuda("cudaSetDevice", err);
  }
  const std::size_t a_bytes = static_cast<std::size_t>(m) * h->view.k * sizeof(float);
  const std::size_t y_bytes = static_cast<std::size_t>(m) * h->view.n * sizeof(float);
  int rc = Grow(reinterpret_cast<void **>(&h->a_dev), &h->a_dev_bytes, a_bytes);
  if (rc != MNB_OK) {
    return rc;
  }
  constexpr std::size_t kDirectLimit = 1u << 20;
  // Where the caller's buffers live is asked once per (A, Y, sizes): two cudaPointerGetAttributes
  // per call cost about as much as a kernel launch. A buffer that is freed and another one
  // page-locked at the same address between two calls of the same sizes is a caller error here.
  if (a_host != h->host_a || y_host != h->host_y || a_bytes != h->host_a_bytes || y_bytes != h->host_y_bytes) {
    cudaPointerAttributes attributes{};
    h->host_a_alias = nullptr;
    h->host_y_alias = nullptr;
    if (a_bytes <= kDirectLimit && (reinterpret_cast<std::uintptr_t>(a_host) & 15u) == 0 &&
        cudaPointerGetAttributes(&attributes, a_host) == cudaSuccess && attributes.type == cudaMemoryTypeHost &&
        attributes.devicePointer != nullptr) {
      h->host_a_alias = static_cast<const float *>(attributes.devicePointer);
    } else {
      cudaGetLastError(); // an unregistered pointer reports an error on some drivers: not a failure here
    }
    if (y_bytes <= kDirectLimit && cudaPointerGetAttributes(&attributes, y_host) == cudaSuccess &&
        attributes.type == cudaMemoryTypeHost && attributes.devicePointer != nullptr) {
      h->host_y_alias = static_cast<float *>(attributes.devicePointer);
    } else {
      cudaGetLastError();
    }
    h->host_a = a_host;
    h->host_y = y_host;
    h->host_a_bytes = a_bytes;
    h->host_y_bytes = y_bytes;
  }
  const float *a_alias = h->host_a_alias;
  if (a_alias != nullptr) {
    const int count16 = static_cast<int>(a_bytes / 16);
    const int tail = static_cast<int>((a_bytes - static_cast<std::size_t>(count16) * 16) / sizeof(float));
    const int threads = count16 > tail ? count16 : tail;
    nbits_fetch_kernel<<<(threads + 255) / 256, 256, 0, h->stream>>>(
        reinterpret_cast<const uint4 *>(a_alias), reinterpret_cast<uint4 *>(h->a_dev), count16,
        a_alias + static_cast<std::size_t>(count16) * 4, h->a_dev + static_cast<std::size_t>(count16) * 4, tail);
    err = cudaGetLastError();
    if (err == cudaSuccess) {
      mnb::CountLaunch();
    }
  } else {
    err = cudaMemcpyAsync(h->a_dev, a_host, a_bytes, cudaMemcpyHostToDevice, h->stream);
  }
  if (err != cudaSuccess) {
    return FailCuda("copy A to device", err);
  }
  // Y: when the caller's buffer is page-locked (cudaHostAlloc / cudaHostRegister) and small (a
  // decode-sized result), the kernels store straight into it through its device alias, which
  // saves a copy launch per call; any other buffer gets a device staging buffer and a
  // device-to-host copy, which keeps the SMs from waiting on the host link for large results.
  float *y_alias = h->host_y_alias;
  if (y_alias == nullptr) {
    rc = Grow(reinterpret_cast<void **>(&h->y_dev), &h->y_dev_bytes, y_bytes);
    if (rc != MNB_OK) {
      return rc;
    }
  }
  OutputView out{y_alias != nullptr ? y_alias : h->y_dev, h->view.n, 0};
  mnb::SetDependentLaunchHint(a_alias != nullptr);
  rc = Dispatch(h, h->a_dev, m, accuracy_level, path, out, h->stream);
  mnb::SetDependentLaunchHint(false);
  if (rc != MNB_OK) {
    return rc;
  }
  if (y_alias == nullptr) {
    err = cudaMemcpyAsync(y_host, h->y_dev, y_bytes, cudaMemcpyDeviceToHost, h->stream);
    if (err != cudaSuccess) {
      return FailCuda("copy Y to host", err);
    }
  }
  err = cudaStreamSynchronize(h->stream);
  if (err != cudaSuccess) {
    return FailCuda("MatMulNBits execution", err);
  }
  const int status = *static_cast<volatile int *>(h->status_host);
  if (status != 0) {
    *h->status_host = 0;
    char text[96];
    std::snprintf(text, sizeof(text), "matmulnbits_b200: device-side wait timed out (status %d).", status);
    return Fail(MNB_ERR_DEVICE_TIMEOUT, text);
  }
  return MNB_OK;
}

int mnb_weights_poll_status(mnb_weights *h, int *status) {
  if (h == nullptr || status == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_weights_poll_status: null argument.");
  }
  std::lock_guard<std::mutex> guard(h->mutex);
  cudaError_t err = cudaSetDevice(h->device);
  if (err == cudaSuccess) {
    err = cudaDeviceSynchronize();
  }
  if (err != cudaSuccess) {
    return FailCuda("status read", err);
  }
  *status = *static_cast<volatile int *>(h->status_host);
  if (*status != 0) {
    *h->status_host = 0;
  }
  return MNB_OK;
}

int mnb_dequant_int_device(mnb_weights *h, int32_t *out_dev, void *stream) {
  if (h == nullptr || out_dev == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_dequant_int_device: null argument.");
  }
  std::lock_guard<std::mutex> guard(h->mutex);
  const cudaError_t err = cudaSetDevice(h->device);
  if (err != cudaSuccess) {
    return FailCuda("cudaSetDevice", err);
  }
  if (mnb::LaunchDequantInt(h->view, out_dev, static_cast<cudaStream_t>(stream)) == nullptr) {
    return FailCuda("dequant launch", cudaGetLastError());
  }
  return MNB_OK;
}

int mnb_quantize_a_device(const float *a_dev, int64_t m, int64_t k, int block_size, int8_t *aq_dev,
                          float *a_scales_dev, void *stream) {
  if (a_dev == nullptr || aq_dev == nullptr || a_scales_dev == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_quantize_a_device: null argument.");
  }
  if (m <= 0 || k <= 0 || block_size < 16 || (block_size & (block_size - 1)) != 0) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_quantize_a_device: bad geometry.");
  }
  if (mnb::LaunchQuantizeA(a_dev, m, k, block_size, aq_dev, a_scales_dev,
                           static_cast<cudaStream_t>(stream)) == nullptr) {
    return FailCuda("quantize launch", cudaGetLastError());
  }
  return MNB_OK;
}

int mnb_int8_block_dots_device(mnb_weights *h, const int8_t *aq_dev, int64_t m, int32_t *dots_dev,
                               void *stream) {
  if (h == nullptr || aq_dev == nullptr || dots_dev == nullptr || m <= 0) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_int8_block_dots_device: bad argument.");
  }
  std::lock_guard<std::mutex> guard(h->mutex);
  const cudaError_t err = cudaSetDevice(h->device);
  if (err != cudaSuccess) {
    return FailCuda("cudaSetDevice", err);
  }
  if (mnb::LaunchInt8BlockDots(h->view, aq_dev, m, dots_dev, static_cast<cudaStream_t>(stream)) ==
      nullptr) {
    return FailCuda("block-dot launch", cudaGetLastError());
  }
  return MNB_OK;
}

int mnb_int8_mma_block_dots_device(mnb_weights *h, const float *a_dev, int64_t m, float *y_dev, int32_t *dots_dev,
                                   void *stream) {
  if (h == nullptr || a_dev == nullptr || y_dev == nullptr || dots_dev == nullptr || m <= 0) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_int8_mma_block_dots_device: bad argument.");
  }
  std::lock_guard<std::mutex> guard(h->mutex);
  const cudaError_t err = cudaSetDevice(h->device);
  if (err != cudaSuccess) {
    return FailCuda("cudaSetDevice", err);
  }
  const std::size_t need = m <= 8 ? mnb::Int8MmaScratchBytes(h->view, m) : 0;
  const char *name = nullptr;
  if (need != 0) {
    const int rc = Grow(&h->scratch_a, &h->scratch_a_bytes, need);
    if (rc != MNB_OK) {
      return rc;
    }
    OutputView out{y_dev, h->view.n, 0};
    name = mnb::LaunchInt8MmaBlockDots(h->view, a_dev, m, static_cast<unsigned char *>(h->scratch_a), out, dots_dev,
                                       h->status_dev, static_cast<cudaStream_t>(stream), h->sm_count);
  }
  if (name == nullptr) {
    return Fail(MNB_ERR_UNSUPPORTED,
                "mnb_int8_mma_block_dots_device: needs M <= 8 and a shape of the integer-MMA path (bits=4, "
                "32 <= block_size <= 1024, packed rows a multiple of 128 bytes).");
  }
  mnb::t_last_kernel = name;
  return MNB_OK;
}

// ---- accuracy_level 4 without any allocation ------------------------------------------------
// The quantized activations and their block scales live in a fixed array inside the library
// image instead of cudaMalloc'ed scratch. Every GPU that loads the library carries the array
// until the process exits.
namespace {
constexpr std::int64_t kStaticMaxTokens = MNB_STATIC_MAX_TOKENS;
constexpr std::int64_t kStaticMaxPaddedK = MNB_STATIC_MAX_PADDED_K;
constexpr std::size_t kStaticAqBytes = static_cast<std::size_t>(kStaticMaxTokens) * kStaticMaxPaddedK;
constexpr std::size_t kStaticScaleBytes =
    static_cast<std::size_t>(kStaticMaxTokens) * (kStaticMaxPaddedK / 16) * sizeof(float);
constexpr int kStaticMaxDevices = 64;
} // namespace

static __device__ __align__(256) unsigned char g_static_scratch[kStaticAqBytes + kStaticScaleBytes];

namespace {
std::mutex g_static_mutex;
std::mutex g_static_launch_mutex;
unsigned char *g_static_address[kStaticMaxDevices] = {};

// In host code `g_static_scratch` is only a handle for the symbol, not a device address: the
// address is looked up once per device, with that device current, and handed to the kernels.
int StaticScratchFor(int device, unsigned char **out) {
  if (device < 0 || device >= kStaticMaxDevices) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_matmul_int8_static: device index out of range.");
  }
  std::lock_guard<std::mutex> guard(g_static_mutex);
  if (g_static_address[device] == nullptr) {
    unsigned char *ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_static_scratch);
    if (err != cudaSuccess) {
      return FailCuda("cudaGetSymbolAddress(static scratch)", err);
    }
    if (ptr == nullptr) {
      return Fail(MNB_ERR_CUDA, "matmulnbits_b200: cudaGetSymbolAddress(static scratch) gave a null address.");
    }
    g_static_address[device] = ptr;
  }
  *out = g_static_address[device];
  return MNB_OK;
}
} // namespace

int mnb_matmul_int8_static(mnb_weights *h, const float *a_dev, int64_t m, float *y_dev, void *stream) {
  if (h == nullptr || a_dev == nullptr || y_dev == nullptr) {
    return Fail(MNB_ERR_INVALID_ARGUMENT, "mnb_matmul_int8_static: null argument.");
  }
  const WeightView &w = h->view;
  const std::int64_t padded_k = static_cast<std::int64_t>(w.n_blocks) * w.block_size;
  if (m < 1 || m > kStaticMaxTokens || padded_k > kStaticMaxPaddedK) {
    char text[200];
    std::snprintf(text, sizeof(text),
                  "mnb_matmul_int8_static: M=%lld, padded K=%lld exceed the built-in scratch "
                  "(M <= %lld, ceil(K/block_size)*block_size <= %lld); use mnb_matmul_device.",
                  static_cast<long long>(m), static_cast<long long>(padded_k),
                  static_cast<long long>(kStaticMaxTokens), static_cast<long long>(kStaticMaxPaddedK));
    return Fail(MNB_ERR_INVALID_ARGUMENT, text);
  }
  std::lock_guard<std::mutex> guard(h->mutex);
  const cudaError_t err = cudaSetDevice(h->device);
  if (err != cudaSuccess) {
    return FailCuda("cudaSetDevice", err);
  }
  int rc = CheckDeviceOperands(h, a_dev, y_dev);
  if (rc != MNB_OK) {
    return rc;
  }
  unsigned char *scratch = nullptr;
  rc = StaticScratchFor(h->device, &scratch);
  if (rc != MNB_OK) {
    return rc;
  }
  // Every byte of the two regions that the matmul reads is rewritten by the quantization
  // kernel of the same call (padding columns included), so nothing has to be cleared.
  std::int8_t *aq = reinterpret_cast<std::int8_t *>(scratch);
  float *a_scales = reinterpret_cast<float *>(scratch + kStaticAqBytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The two launches of a call are queued as a pair: another host thread (another handle, the
  // same stream) must not get its quantization between this call's quantization and product.
  std::lock_guard<std::mutex> pair_guard(g_static_launch_mutex);
  const char *name = mnb::LaunchQuantizeAPadded(a_dev, m, w.k, w.block_size, aq, a_scales, s);
  if (name != nullptr) {
    OutputView out{y_dev, w.n, 0};
    name = mnb::LaunchInt8Matmul(w, aq, a_scales, m, out, s, h->sm_count);
  }
  if (name == nullptr) {
    return Fail(MNB_ERR_UNSUPPORTED,
                "mnb_matmul_int8_static: needs packed rows and a weight base aligned to eight codes (4 bytes "
                "for 4-bit, 8 bytes for 8-bit weights).");
  }
  mnb::t_last_kernel = name;
  return MNB_OK;
}

int64_t mnb_launch_count(void) { return mnb::g_launches.load(std::memory_order_relaxed); }

const char *mnb_last_kernel(void) { return mnb::t_last_kernel; }

int64_t mnb_weights_n(const mnb_weights *h) { return h != nullptr ? h->view.n : 0; }
int64_t mnb_weights_k(const mnb_weights *h) { return h != nullptr ? h->view.k : 0; }
int mnb_weights_bits(const mnb_weights *h) { return h != nullptr ? h->view.bits : 0; }
int mnb_weights_block_size(const mnb_weights *h) { return h != nullptr ? h->view.block_size : 0; }

} // extern "C"
