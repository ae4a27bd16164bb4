// Decode path of MatMulNBits for sm_100a: fused unpack -> dequantize -> GEMV on CUDA cores.
//
// Two kernels:
//   * nbits_gemv_stream_kernel - persistent, one CTA per SM. A producer warp streams whole
//     row tiles of the packed weights (plus their scales and zero points) into a ring of
//     shared-memory stages with 1-D bulk (TMA) copies completed on mbarriers; 16 consumer
//     warps read 128-bit chunks from shared memory, turn nibbles/bytes into fp32 with a
//     magic-number OR (no integer->float conversion instruction), multiply-accumulate with
//     packed fp32x2 FMAs against activations held in registers, and reduce with warp
//     shuffles. Memory-bound by design: every weight byte is read from HBM exactly once.
//   * nbits_gemv_generic_kernel - one warp per output column, scalar code, any shape. Used
//     for shapes the streaming kernel does not take (unaligned rows, block_size 16, ...).
//
// The arithmetic is the partition the reference uses for its skinny-M GEMV - stream B once,
// split N across workers (onnx_light_cpu/impl/math/gemm_kernel.cc:1219-1258) - with the
// packed-INT4 conventions of onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:60-93.
//
// Numerics: q is exact in fp32; sum_k a_k*q_k is accumulated in fp32 per 32-element chunk,
// then (chunk_sum - zp * sum_k a_k) * scale is added to the row accumulator. Differences
// from a sequential fp32 sum are summation-order only.

#include "nbits_common.cuh"
#include "nbits_ptx.cuh"

#include <cstdint>

namespace mnb {
namespace {

constexpr int kConsumerThreads = 512;
constexpr int kConsumerWarps = kConsumerThreads / 32;
constexpr int kProducerThreads = 32;
constexpr int kRowsPerThread = 4;
constexpr int kMaxStages = 4;
constexpr int kChunkBytes = 16;

struct StreamParams {
  WeightView w;
  const float *a;
  int m_total;
  OutputView out;
  int *status;
  int cc_log2;        // log2(chunk columns handled by one row group)
  int row_groups;     // kConsumerThreads >> cc_log2
  int tile_rows;      // row_groups * kRowsPerThread
  int chunks_per_row; // row_bytes / 16
  int rows_per_cta;
  int stages;
  int stage_b_bytes;     // tile_rows * row_bytes
  int stage_scale_bytes; // tile_rows * n_blocks * 4, rounded up to 16
  int stage_zp_bytes;    // tile_rows * zp_row_bytes rounded up to 16 (0 without zero points)
  int stage_bytes;
  int block_shift; // log2(block_size)
};

__device__ __forceinline__ float2 Ffma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 Fadd2(float2 a, float2 b) { return __fadd2_rn(a, b); }

// Reduces V per-thread values over the 32 lanes of a warp with V-1 + log2(32/V) shuffles.
// On return, value index ((lane * V) >> 5) is complete in every lane; the function returns it.
template <int V> __device__ __forceinline__ float WarpMultiReduce(float (&v)[V], int lane) {
  static_assert(V == 1 || V == 2 || V == 4 || V == 8 || V == 16, "V must be a power of two");
  int width = V;
  int offset = 16;
#pragma unroll
  for (int step = 0; step < 5; ++step) {
    if (width > 1) {
      const bool upper = (lane & offset) != 0;
      const int half = width >> 1;
#pragma unroll
      for (int i = 0; i < V / 2; ++i) {
        if (i < half) {
          const float send = upper ? v[i] : v[i + half];
          const float keep = upper ? v[i + half] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, offset);
        }
      }
      width = half;
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], offset);
    }
    offset >>= 1;
  }
  return v[0];
}

// Per-thread activation registers for one chunk column: 32 (4-bit) or 16 (8-bit) consecutive
// k, pre-multiplied by the power of two that undoes the bit position of their code.
template <int BITS> struct ChunkTraits;
template <> struct ChunkTraits<4> {
  static constexpr int kWeights = 32;
};
template <> struct ChunkTraits<8> {
  static constexpr int kWeights = 16;
};

// sum_e a[e] * code[e] for one 16-byte chunk. `ap` holds the pre-scaled activations as pairs.
template <int BITS>
__device__ __forceinline__ float ChunkDot(const uint4 &q, const float2 *ap) {
  const float2 kMagic2 = make_float2(-8388608.0f, -8388608.0f);
  float2 acc0 = make_float2(0.0f, 0.0f);
  float2 acc1 = make_float2(0.0f, 0.0f);
  const std::uint32_t words[4] = {q.x, q.y, q.z, q.w};
  if constexpr (BITS == 4) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const std::uint32_t w = words[i];
      const std::uint32_t hi = w >> 12;
      // nibble j sits at bit 4j of w (j <= 4) or at bit 4(j-3) of hi (j >= 5)
      const float x0 = __uint_as_float((w & 0x0000000fu) | 0x4b000000u);
      const float x1 = __uint_as_float((w & 0x000000f0u) | 0x4b000000u);
      const float x2 = __uint_as_float((w & 0x00000f00u) | 0x4b000000u);
      const float x3 = __uint_as_float((w & 0x0000f000u) | 0x4b000000u);
      const float x4 = __uint_as_float((w & 0x000f0000u) | 0x4b000000u);
      const float x5 = __uint_as_float((hi & 0x00000f00u) | 0x4b000000u);
      const float x6 = __uint_as_float((hi & 0x0000f000u) | 0x4b000000u);
      const float x7 = __uint_as_float((hi & 0x000f0000u) | 0x4b000000u);
      acc0 = Ffma2(Fadd2(make_float2(x0, x1), kMagic2), ap[4 * i + 0], acc0);
      acc1 = Ffma2(Fadd2(make_float2(x2, x3), kMagic2), ap[4 * i + 1], acc1);
      acc0 = Ffma2(Fadd2(make_float2(x4, x5), kMagic2), ap[4 * i + 2], acc0);
      acc1 = Ffma2(Fadd2(make_float2(x6, x7), kMagic2), ap[4 * i + 3], acc1);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const std::uint32_t w = words[i];
      const float x0 = __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7540));
      const float x1 = __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7541));
      const float x2 = __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7542));
      const float x3 = __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7543));
      acc0 = Ffma2(Fadd2(make_float2(x0, x1), kMagic2), ap[2 * i + 0], acc0);
      acc1 = Ffma2(Fadd2(make_float2(x2, x3), kMagic2), ap[2 * i + 1], acc1);
    }
  }
  const float2 s = Fadd2(acc0, acc1);
  return s.x + s.y;
}

// Pre-scale factor for element e of a chunk (undoes the bit position left in place by the OR).
template <int BITS> __device__ __forceinline__ float PrescaleOf(int e) {
  if constexpr (BITS == 8) {
    return 1.0f;
  } else {
    const int j = e & 7;
    const int pos = j <= 4 ? j : j - 3; // in nibbles
    return 1.0f / static_cast<float>(1 << (4 * pos));
  }
}

template <int BITS, int MT, int J>
__global__ void __launch_bounds__(kConsumerThreads + kProducerThreads, 1)
    nbits_gemv_stream_kernel(const StreamParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int kW = ChunkTraits<BITS>::kWeights;
  constexpr int kV = kRowsPerThread * MT;

  // shared memory carve-up: [stages x (B | scales | zp)] [barriers] [reduction scratch]
  unsigned char *stage_base = smem_raw;
  std::uint64_t *full_bar =
      reinterpret_cast<std::uint64_t *>(smem_raw + static_cast<size_t>(p.stages) * p.stage_bytes);
  std::uint64_t *empty_bar = full_bar + kMaxStages;
  float *red = reinterpret_cast<float *>(empty_bar + kMaxStages); // [2][row_groups][kV][wpg]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const bool is_producer = warp == kConsumerWarps;

  const std::int64_t row_begin = static_cast<std::int64_t>(blockIdx.x) * p.rows_per_cta;
  std::int64_t rows_here = p.w.n - row_begin;
  if (rows_here > p.rows_per_cta) {
    rows_here = p.rows_per_cta;
  }
  if (rows_here < 0) {
    rows_here = 0;
  }
  const int num_tiles = static_cast<int>((rows_here + p.tile_rows - 1) / p.tile_rows);
  const int m_base = blockIdx.y * MT;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      ptx::MbarInit(&full_bar[s], kProducerThreads);
      ptx::MbarInit(&empty_bar[s], kConsumerWarps);
    }
    ptx::FenceMbarInit();
  }
  __syncthreads();

  if (is_producer) {
    // ---------------- producer warp: fill the stage ring ----------------
    for (int t = 0; t < num_tiles; ++t) {
      const int s = t % p.stages;
      const std::uint32_t round = static_cast<std::uint32_t>(t / p.stages);
      if (!ptx::MbarWait(&empty_bar[s], (round & 1u) ^ 1u)) {
        if (lane == 0) {
          atomicExch(p.status, kDeviceTimeoutEmptyBarrier);
        }
        break;
      }
      const std::int64_t row0 = row_begin + static_cast<std::int64_t>(t) * p.tile_rows;
      std::int64_t rows = rows_here - static_cast<std::int64_t>(t) * p.tile_rows;
      if (rows > p.tile_rows) {
        rows = p.tile_rows;
      }
      unsigned char *sb = stage_base + static_cast<size_t>(s) * p.stage_bytes;
      unsigned char *ss = sb + p.stage_b_bytes;
      unsigned char *sz = ss + p.stage_scale_bytes;

      const std::uint32_t b_bytes = static_cast<std::uint32_t>(rows) * p.w.row_bytes;
      const float *scale_src = p.w.scales + row0 * p.w.n_blocks;
      const std::uint32_t scale_bytes = static_cast<std::uint32_t>(rows) * p.w.n_blocks * 4u;
      const bool scale_bulk =
          ((reinterpret_cast<std::uintptr_t>(scale_src) | scale_bytes) & 15u) == 0;
      const std::uint8_t *zp_src = p.w.zp != nullptr ? p.w.zp + row0 * p.w.zp_row_bytes : nullptr;
      const std::uint32_t zp_bytes =
          p.w.zp != nullptr ? static_cast<std::uint32_t>(rows) * p.w.zp_row_bytes : 0u;
      const bool zp_bulk =
          zp_bytes != 0 && ((reinterpret_cast<std::uintptr_t>(zp_src) | zp_bytes) & 15u) == 0;

      if (!scale_bulk) {
        float *dst = reinterpret_cast<float *>(ss);
        for (std::uint32_t i = lane; i < scale_bytes / 4u; i += 32) {
          dst[i] = scale_src[i];
        }
      }
      if (zp_bytes != 0 && !zp_bulk) {
        for (std::uint32_t i = lane; i < zp_bytes; i += 32) {
          sz[i] = zp_src[i];
        }
      }
      if (lane == 0) {
        const std::uint32_t tx =
            b_bytes + (scale_bulk ? scale_bytes : 0u) + (zp_bulk ? zp_bytes : 0u);
        ptx::MbarArriveExpectTx(&full_bar[s], tx);
        ptx::BulkLoad(sb, p.w.b + row0 * p.w.row_bytes, b_bytes, &full_bar[s]);
        if (scale_bulk) {
          ptx::BulkLoad(ss, scale_src, scale_bytes, &full_bar[s]);
        }
        if (zp_bulk) {
          ptx::BulkLoad(sz, zp_src, zp_bytes, &full_bar[s]);
        }
      } else {
        ptx::MbarArrive(&full_bar[s]);
      }
    }
    // Do not leave while bulk copies may still be landing in this CTA's shared memory: wait
    // (bounded) until the consumers have drained every stage that was filled.
    for (int t = num_tiles - p.stages < 0 ? 0 : num_tiles - p.stages; t < num_tiles; ++t) {
      const int s = t % p.stages;
      const std::uint32_t round = static_cast<std::uint32_t>(t / p.stages);
      if (!ptx::MbarWait(&empty_bar[s], round & 1u)) {
        break;
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  const int cc = tid & ((1 << p.cc_log2) - 1);
  const int rg = tid >> p.cc_log2;
  const int warps_per_group = (1 << p.cc_log2) >> 5; // chunk columns per group >= 32
  const int warp_in_group = warp & (warps_per_group - 1);

  // activations of this thread's chunk columns, pre-scaled, as pairs; and their plain sums
  float2 ap[MT][J][kW / 2];
  float a_sum[MT][J];
#pragma unroll
  for (int mi = 0; mi < MT; ++mi) {
    const int m = m_base + mi;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = cc + (j << p.cc_log2);
      const std::int64_t k0 = static_cast<std::int64_t>(c) * kW;
      float total = 0.0f;
#pragma unroll
      for (int e = 0; e < kW; e += 2) {
        float v0 = 0.0f, v1 = 0.0f;
        if (m < p.m_total && c < p.chunks_per_row) {
          if (k0 + e < p.w.k) {
            v0 = __ldg(p.a + static_cast<std::int64_t>(m) * p.w.k + k0 + e);
          }
          if (k0 + e + 1 < p.w.k) {
            v1 = __ldg(p.a + static_cast<std::int64_t>(m) * p.w.k + k0 + e + 1);
          }
        }
        total += v0 + v1;
        ap[mi][j][e / 2] = make_float2(v0 * PrescaleOf<BITS>(e), v1 * PrescaleOf<BITS>(e + 1));
      }
      a_sum[mi][j] = total;
    }
  }

  const int default_zp = 1 << (BITS - 1);
  const bool has_zp = p.w.zp != nullptr;

  for (int t = 0; t < num_tiles; ++t) {
    const int s = t % p.stages;
    const std::uint32_t round = static_cast<std::uint32_t>(t / p.stages);
    if (!ptx::MbarWait(&full_bar[s], round & 1u)) {
      atomicExch(p.status, kDeviceTimeoutFullBarrier);
      return;
    }
    const unsigned char *sb = stage_base + static_cast<size_t>(s) * p.stage_bytes;
    const float *ss = reinterpret_cast<const float *>(sb + p.stage_b_bytes);
    const unsigned char *sz = sb + p.stage_b_bytes + p.stage_scale_bytes;
    std::int64_t rows = rows_here - static_cast<std::int64_t>(t) * p.tile_rows;
    if (rows > p.tile_rows) {
      rows = p.tile_rows;
    }

    float acc[kV];
#pragma unroll
    for (int v = 0; v < kV; ++v) {
      acc[v] = 0.0f;
    }
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
      const int r = rg * kRowsPerThread + i;
      if (r < rows) {
#pragma unroll
        for (int j = 0; j < J; ++j) {
          const int c = cc + (j << p.cc_log2);
          if (c < p.chunks_per_row) {
            const uint4 q = *reinterpret_cast<const uint4 *>(sb + static_cast<size_t>(r) * p.w.row_bytes +
                                                             static_cast<size_t>(c) * kChunkBytes);
            const int block = (c * kW) >> p.block_shift;
            const float scale = ss[r * p.w.n_blocks + block];
            int zp = default_zp;
            if (has_zp) {
              if constexpr (BITS == 8) {
                zp = sz[r * p.w.zp_row_bytes + block];
              } else {
                const int byte = sz[r * p.w.zp_row_bytes + (block >> 1)];
                zp = (block & 1) ? (byte >> 4) : (byte & 0x0f);
              }
            }
            const float zpf = static_cast<float>(zp);
#pragma unroll
            for (int mi = 0; mi < MT; ++mi) {
              const float raw = ChunkDot<BITS>(q, ap[mi][j]);
              acc[i * MT + mi] = fmaf(scale, fmaf(-zpf, a_sum[mi][j], raw), acc[i * MT + mi]);
            }
          }
        }
      }
    }
    // stage no longer needed by this warp
    __syncwarp();
    if (lane == 0) {
      ptx::MbarArrive(&empty_bar[s]);
    }

    // reduce over the chunk columns of the row group
    const float mine = WarpMultiReduce<kV>(acc, lane);
    const int value_index = (lane * kV) >> 5; // = i * MT + mi
    const bool writer_lane = (lane & (32 / kV - 1)) == 0;
    const std::int64_t row0 = row_begin + static_cast<std::int64_t>(t) * p.tile_rows;
    if (warps_per_group == 1) {
      if (writer_lane) {
        const int i = value_index / MT;
        const int mi = value_index % MT;
        const int r = rg * kRowsPerThread + i;
        const int m = m_base + mi;
        if (r < rows && m < p.m_total) {
          const std::int64_t col = row0 + r;
          const float bias = p.w.bias != nullptr ? p.w.bias[col] : 0.0f;
          p.out.y[static_cast<std::int64_t>(m) * p.out.ld + p.out.col_offset + col] = mine + bias;
        }
      }
    } else {
      float *buf = red + static_cast<size_t>(t & 1) * p.row_groups * kV * warps_per_group +
                   static_cast<size_t>(rg) * kV * warps_per_group;
      if (writer_lane) {
        buf[value_index * warps_per_group + warp_in_group] = mine;
      }
      // named barrier over the threads of this row group only (ids 1..8; 0 is __syncthreads)
      asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(1 << p.cc_log2) : "memory");
      if (cc < kV) {
        float total = 0.0f;
        for (int wg = 0; wg < warps_per_group; ++wg) {
          total += buf[cc * warps_per_group + wg];
        }
        const int i = cc / MT;
        const int mi = cc % MT;
        const int r = rg * kRowsPerThread + i;
        const int m = m_base + mi;
        if (r < rows && m < p.m_total) {
          const std::int64_t col = row0 + r;
          const float bias = p.w.bias != nullptr ? p.w.bias[col] : 0.0f;
          p.out.y[static_cast<std::int64_t>(m) * p.out.ld + p.out.col_offset + col] = total + bias;
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Generic kernel: one warp per output column, any geometry.
constexpr int kGenericMaxM = 16;

__global__ void __launch_bounds__(256)
    nbits_gemv_generic_kernel(const WeightView w, const float *a, int m_total, OutputView out) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const std::int64_t col = static_cast<std::int64_t>(blockIdx.x) * 8 + warp;
  const int m_base = blockIdx.y * kGenericMaxM;
  if (col >= w.n) {
    return;
  }
  float acc[kGenericMaxM];
#pragma unroll
  for (int mi = 0; mi < kGenericMaxM; ++mi) {
    acc[mi] = 0.0f;
  }
  for (int block = 0; block < w.n_blocks; ++block) {
    const float scale = w.scales[col * w.n_blocks + block];
    const int zp = ZeroPointOf(w, col, block);
    const std::int64_t k0 = static_cast<std::int64_t>(block) * w.block_size;
    for (int e = lane; e < w.block_size; e += 32) {
      const std::int64_t kk = k0 + e;
      if (kk < w.k) {
        const float wv = static_cast<float>(CodeOf(w, col, kk) - zp) * scale;
#pragma unroll
        for (int mi = 0; mi < kGenericMaxM; ++mi) {
          if (m_base + mi < m_total) {
            acc[mi] = fmaf(a[static_cast<std::int64_t>(m_base + mi) * w.k + kk], wv, acc[mi]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int mi = 0; mi < kGenericMaxM; ++mi) {
    float v = acc[mi];
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      v += __shfl_xor_sync(0xffffffffu, v, offset);
    }
    if (lane == 0 && m_base + mi < m_total) {
      const float bias = w.bias != nullptr ? w.bias[col] : 0.0f;
      out.y[static_cast<std::int64_t>(m_base + mi) * out.ld + out.col_offset + col] = v + bias;
    }
  }
}

int Log2Exact(int v) {
  int l = 0;
  while ((1 << l) < v) {
    ++l;
  }
  return l;
}

template <int BITS, int MT, int J>
cudaError_t LaunchStreamInstance(const StreamParams &p, dim3 grid, size_t smem, cudaStream_t stream) {
  auto kernel = nbits_gemv_stream_kernel<BITS, MT, J>;
  cudaError_t err =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) {
    return err;
  }
  kernel<<<grid, kConsumerThreads + kProducerThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

} // namespace

const char *LaunchGemvStream(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                             int *status_word, cudaStream_t stream, int sm_count) {
  if (m < 1 || m > 16 || w.n < 1 || w.k < 1) {
    return nullptr;
  }
  if ((w.row_bytes % kChunkBytes) != 0 || (reinterpret_cast<std::uintptr_t>(w.b) & 15u) != 0) {
    return nullptr;
  }
  if (w.bits == 4 && w.block_size < 32) {
    return nullptr; // a 16-byte chunk must lie inside one quantization block
  }
  const int chunks_per_row = w.row_bytes / kChunkBytes;
  if (chunks_per_row > 2 * kConsumerThreads) {
    return nullptr;
  }
  StreamParams p{};
  p.w = w;
  p.a = a;
  p.m_total = static_cast<int>(m);
  p.out = out;
  p.status = status_word;
  p.chunks_per_row = chunks_per_row;
  int cc = 32;
  while (cc < chunks_per_row && cc < kConsumerThreads) {
    cc <<= 1;
  }
  p.cc_log2 = Log2Exact(cc);
  p.row_groups = kConsumerThreads / cc;
  p.tile_rows = p.row_groups * kRowsPerThread;
  const int j = (chunks_per_row + cc - 1) / cc;
  p.block_shift = Log2Exact(w.block_size);
  p.stage_b_bytes = p.tile_rows * w.row_bytes;
  p.stage_scale_bytes = (p.tile_rows * w.n_blocks * 4 + 15) & ~15;
  p.stage_zp_bytes = w.zp != nullptr ? ((p.tile_rows * w.zp_row_bytes + 15) & ~15) : 0;
  p.stage_bytes = (p.stage_b_bytes + p.stage_scale_bytes + p.stage_zp_bytes + 127) & ~127;
  const int warps_per_group = cc / 32;
  const size_t tail_bytes = 2 * kMaxStages * sizeof(std::uint64_t) +
                            static_cast<size_t>(2) * p.row_groups * kRowsPerThread * 2 * warps_per_group * sizeof(float);
  const size_t budget = 200 * 1024;
  int stages = static_cast<int>((budget - tail_bytes) / static_cast<size_t>(p.stage_bytes));
  if (stages > kMaxStages) {
    stages = kMaxStages;
  }
  if (stages < 2) {
    return nullptr;
  }
  p.stages = stages;
  const size_t smem = static_cast<size_t>(stages) * p.stage_bytes + tail_bytes;

  int ctas = sm_count > 0 ? sm_count : 148;
  const std::int64_t max_ctas = (w.n + p.tile_rows - 1) / p.tile_rows;
  if (ctas > max_ctas) {
    ctas = static_cast<int>(max_ctas);
  }
  p.rows_per_cta = static_cast<int>((w.n + ctas - 1) / ctas);

  const int mt = (m == 1 || j == 2) ? 1 : 2; // two chunk columns x two rows of A would spill
  dim3 grid(static_cast<unsigned>(ctas), static_cast<unsigned>((m + mt - 1) / mt), 1);
  cudaError_t err = cudaErrorInvalidValue;
  const char *name = nullptr;
#define MNB_STREAM_CASE(B_, M_, J_)                                                              \
  if (w.bits == B_ && mt == M_ && j == J_) {                                                     \
    err = LaunchStreamInstance<B_, M_, J_>(p, grid, smem, stream);                               \
    name = "nbits_gemv_stream_kernel<" #B_ "," #M_ "," #J_ ">";                                  \
  }
  MNB_STREAM_CASE(4, 1, 1)
  MNB_STREAM_CASE(4, 2, 1)
  MNB_STREAM_CASE(4, 1, 2)
  MNB_STREAM_CASE(8, 1, 1)
  MNB_STREAM_CASE(8, 2, 1)
  MNB_STREAM_CASE(8, 1, 2)
#undef MNB_STREAM_CASE
  if (err != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return name;
}

const char *LaunchGemvGeneric(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                              cudaStream_t stream) {
  if (m < 1 || w.n < 1) {
    return nullptr;
  }
  dim3 grid(static_cast<unsigned>((w.n + 7) / 8),
            static_cast<unsigned>((m + kGenericMaxM - 1) / kGenericMaxM), 1);
  nbits_gemv_generic_kernel<<<grid, 256, 0, stream>>>(w, a, static_cast<int>(m), out);
  if (cudaGetLastError() != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return "nbits_gemv_generic_kernel";
}

} // namespace mnb
