// Decode path of MatMulNBits for sm_100a: fused unpack -> dequantize -> GEMV on CUDA cores.
//
// Two kernels:
//   * nbits_gemv_stream_kernel - persistent, one CTA per SM. A producer warp streams whole
//     row tiles of the packed weights (plus their scales and zero points) into a ring of
//     shared-memory stages with 1-D bulk (TMA) copies completed on mbarriers. Eight consumer
//     warps each own a few rows of the tile: a warp walks its rows across all of K, reading
//     128-bit chunks from shared memory, turning nibbles/bytes into fp32 with one LOP3 per
//     code (magic-number OR, no integer->float conversion), and accumulating with packed
//     fp32x2 add/fma against the activations, which are staged once per CTA in shared memory
//     (pre-scaled, bank-conflict-free swizzle) and reused across the warp's rows. Warps never
//     wait for one another: the only cross-warp objects are the stage barriers. The row sums
//     are reduced with warp shuffles and written straight to Y.
//     Memory-bound by design: every weight byte is read from HBM exactly once.
//   * nbits_gemv_generic_kernel - one warp per output column, scalar code, any shape. Used
//     for shapes the streaming kernel does not take (unaligned rows, block_size 16, ...).
//
// The arithmetic is the partition the reference uses for its skinny-M GEMV - stream B once,
// split N across workers (onnx_light_cpu/impl/math/gemm_kernel.cc:1219-1258) - with the
// packed-INT4 conventions of onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:60-93.
//
// Numerics: q is exact in fp32; sum_k a_k*q_k is accumulated in fp32 per 16-byte chunk,
// then scale * (chunk_sum - zp * sum_k a_k) is added to the row accumulator. Differences
// from a sequential fp32 sum are summation-order only.

#include "nbits_common.cuh"
#include "nbits_ptx.cuh"

#include <cstdint>

namespace mnb {
namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kProducerThreads = 32;
constexpr int kThreads = kConsumerThreads + kProducerThreads;
constexpr int kMaxStages = 4;
constexpr int kChunkBytes = 16;
constexpr std::uint32_t kMagicBits = 0x4b000000u; // 2^23 as fp32

struct StreamParams {
  WeightView w;
  const float *a;
  int m_total;
  OutputView out;
  int *status;
  int chunks_per_row;   // row_bytes / 16
  int chunk_iters;      // ceil(chunks_per_row / 32): chunk columns per lane
  int rows_per_warp;    // 4, 2 or 1
  int tile_rows;        // kConsumerWarps * rows_per_warp
  int rows_per_cta;
  int stages;
  int stage_b_bytes;     // tile_rows * row_bytes
  int stage_scale_bytes; // tile_rows * n_blocks * 4, rounded up to 16
  int stage_zp_bytes;    // tile_rows * zp_row_bytes rounded up to 16 (0 without zero points)
  int stage_bytes;
  int a_bytes;           // activation staging: MT * chunk_iters * 32 chunks * 128 B (+ sums)
  int block_shift;       // log2(block_size)
  std::uint32_t magic;   // kMagicBits, passed at run time so that it stays in a register
};

// d = (a & mask) | c in one LOP3 (truth table 0xEA).
template <std::uint32_t MASK>
__device__ __forceinline__ std::uint32_t AndOr(std::uint32_t a, std::uint32_t c) {
  std::uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "n"(MASK), "r"(c));
  return d;
}

// acc += ((x0, x1) - 2^23) * ap   with packed fp32x2 instructions.
__device__ __forceinline__ void PairFma(std::uint64_t &acc, std::uint32_t x0, std::uint32_t x1,
                                        std::uint64_t neg_magic2, std::uint64_t ap) {
  asm("{\n\t"
      ".reg .b64 t;\n\t"
      "mov.b64 t, {%1, %2};\n\t"
      "add.rn.f32x2 t, t, %3;\n\t"
      "fma.rn.f32x2 %0, t, %4, %0;\n\t"
      "}"
      : "+l"(acc)
      : "r"(x0), "r"(x1), "l"(neg_magic2), "l"(ap));
}

__device__ __forceinline__ float PairSum(std::uint64_t a, std::uint64_t b) {
  std::uint64_t s;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(s) : "l"(a), "l"(b));
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(s));
  return lo + hi;
}

template <int BITS> struct ChunkTraits;
template <> struct ChunkTraits<4> {
  static constexpr int kWeights = 32; // codes per 16-byte chunk
  static constexpr int kPairs = 16;   // activation pairs per chunk
  static constexpr int kUnits = 8;    // 16-byte units of fp32 activations per chunk
};
template <> struct ChunkTraits<8> {
  static constexpr int kWeights = 16;
  static constexpr int kPairs = 8;
  static constexpr int kUnits = 4;
};

// sum_e a[e] * code[e] for one 16-byte chunk; `ap` holds pre-scaled activation pairs.
template <int BITS>
__device__ __forceinline__ float ChunkDot(const uint4 &q, const std::uint64_t *ap,
                                          std::uint32_t magic, std::uint64_t neg_magic2) {
  std::uint64_t acc0 = 0, acc1 = 0, acc2 = 0, acc3 = 0;
  const std::uint32_t words[4] = {q.x, q.y, q.z, q.w};
  if constexpr (BITS == 4) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const std::uint32_t w = words[i];
      const std::uint32_t hi = w >> 12;
      // code j sits at bit 4j of w (j <= 4) or at bit 4(j-3) of hi (j >= 5); the bit position
      // is undone by the power-of-two pre-scale of the matching activation
      PairFma(acc0, AndOr<0x0000000fu>(w, magic), AndOr<0x000000f0u>(w, magic), neg_magic2, ap[4 * i + 0]);
      PairFma(acc1, AndOr<0x00000f00u>(w, magic), AndOr<0x0000f000u>(w, magic), neg_magic2, ap[4 * i + 1]);
      PairFma(acc2, AndOr<0x000f0000u>(w, magic), AndOr<0x00000f00u>(hi, magic), neg_magic2, ap[4 * i + 2]);
      PairFma(acc3, AndOr<0x0000f000u>(hi, magic), AndOr<0x000f0000u>(hi, magic), neg_magic2, ap[4 * i + 3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const std::uint32_t w = words[i];
      if (i & 1) {
        PairFma(acc2, __byte_perm(w, magic, 0x7540), __byte_perm(w, magic, 0x7541), neg_magic2, ap[2 * i + 0]);
        PairFma(acc3, __byte_perm(w, magic, 0x7542), __byte_perm(w, magic, 0x7543), neg_magic2, ap[2 * i + 1]);
      } else {
        PairFma(acc0, __byte_perm(w, magic, 0x7540), __byte_perm(w, magic, 0x7541), neg_magic2, ap[2 * i + 0]);
        PairFma(acc1, __byte_perm(w, magic, 0x7542), __byte_perm(w, magic, 0x7543), neg_magic2, ap[2 * i + 1]);
      }
    }
  }
  std::uint64_t s01, s23;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(s01) : "l"(acc0), "l"(acc1));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(s23) : "l"(acc2), "l"(acc3));
  return PairSum(s01, s23);
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

// Reduces V per-thread values over the 32 lanes of a warp with V-1 + log2(32/V) shuffles.
// Afterwards value index (lane * V) >> 5 is complete in every lane and is returned.
template <int V, int OFFSET = 16> __device__ __forceinline__ float WarpMultiReduce(float *v, int lane) {
  if constexpr (OFFSET == 0) {
    return v[0];
  } else if constexpr (V > 1) {
    const bool upper = (lane & OFFSET) != 0;
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      const float send = upper ? v[i] : v[i + V / 2];
      const float keep = upper ? v[i + V / 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, OFFSET);
    }
    return WarpMultiReduce<V / 2, OFFSET / 2>(v, lane);
  } else {
    v[0] += __shfl_xor_sync(0xffffffffu, v[0], OFFSET);
    return WarpMultiReduce<1, OFFSET / 2>(v, lane);
  }
}

// Shared-memory position (in bytes) of 16-byte unit `unit` of the pre-scaled activations: rows
// of 128 bytes with the unit index XOR-swizzled by the row, so that lanes reading the same
// unit of consecutive chunks hit different banks.
__device__ __forceinline__ int ActUnitOffset(int unit) {
  const int row = unit >> 3;
  return (row << 7) + (((unit & 7) ^ (row & 7)) << 4);
}

template <int BITS, int MT, int RPW>
__global__ void __launch_bounds__(kThreads, 1) nbits_gemv_stream_kernel(const StreamParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  using Traits = ChunkTraits<BITS>;
  constexpr int kW = Traits::kWeights;
  constexpr int kV = RPW * MT;

  // shared memory: [stages x (B | scales | zp)] [activations: MT x (units | sums)] [barriers]
  unsigned char *stage_base = smem_raw;
  unsigned char *act_base = smem_raw + static_cast<size_t>(p.stages) * p.stage_bytes;
  std::uint64_t *full_bar = reinterpret_cast<std::uint64_t *>(act_base + p.a_bytes);
  std::uint64_t *empty_bar = full_bar + kMaxStages;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const bool is_producer = warp == kConsumerWarps;
  const int chunk_slots = p.chunk_iters * 32;            // chunk columns incl. padding
  const int act_row_bytes = chunk_slots * Traits::kUnits * 16; // pre-scaled activations of one m
  const int act_m_bytes = act_row_bytes + chunk_slots * 4; // + per-chunk plain sums

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
          ReportStatus(p.status, kDeviceTimeoutEmptyBarrier);
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
      const bool scale_bulk = ((reinterpret_cast<std::uintptr_t>(scale_src) | scale_bytes) & 15u) == 0;
      const std::uint8_t *zp_src = p.w.zp != nullptr ? p.w.zp + row0 * p.w.zp_row_bytes : nullptr;
      const std::uint32_t zp_bytes =
          p.w.zp != nullptr ? static_cast<std::uint32_t>(rows) * p.w.zp_row_bytes : 0u;
      const bool zp_bulk = zp_bytes != 0 && ((reinterpret_cast<std::uintptr_t>(zp_src) | zp_bytes) & 15u) == 0;

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
        const std::uint32_t tx = b_bytes + (scale_bulk ? scale_bytes : 0u) + (zp_bulk ? zp_bytes : 0u);
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
  // Stage the activations once: pre-scaled, swizzled, zero beyond K; plus per-chunk sums.
  for (int mi = 0; mi < MT; ++mi) {
    const int m = m_base + mi;
    unsigned char *dst = act_base + mi * act_m_bytes;
    const int units = chunk_slots * Traits::kUnits;
    for (int u = tid; u < units; u += kConsumerThreads) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const std::int64_t kk = static_cast<std::int64_t>(u) * 4 + e;
        const float raw = (m < p.m_total && kk < p.w.k) ? __ldg(p.a + static_cast<std::int64_t>(m) * p.w.k + kk) : 0.0f;
        v[e] = raw * PrescaleOf<BITS>(static_cast<int>(kk & 7));
      }
      *reinterpret_cast<float4 *>(dst + ActUnitOffset(u)) = make_float4(v[0], v[1], v[2], v[3]);
    }
    float *sums = reinterpret_cast<float *>(dst + act_row_bytes);
    for (int c = tid; c < chunk_slots; c += kConsumerThreads) {
      float total = 0.0f;
      for (int e = 0; e < kW; ++e) {
        const std::int64_t kk = static_cast<std::int64_t>(c) * kW + e;
        if (m < p.m_total && kk < p.w.k) {
          total += __ldg(p.a + static_cast<std::int64_t>(m) * p.w.k + kk);
        }
      }
      sums[c] = total;
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); // consumers only

  const std::uint32_t magic = p.magic;
  std::uint64_t neg_magic2;
  {
    const float neg = -__uint_as_float(magic);
    asm("mov.b64 %0, {%1, %1};" : "=l"(neg_magic2) : "f"(neg));
  }
  const int default_zp = 1 << (BITS - 1);
  const bool has_zp = p.w.zp != nullptr;

  for (int t = 0; t < num_tiles; ++t) {
    const int s = t % p.stages;
    const std::uint32_t round = static_cast<std::uint32_t>(t / p.stages);
    std::int64_t rows = rows_here - static_cast<std::int64_t>(t) * p.tile_rows;
    if (rows > p.tile_rows) {
      rows = p.tile_rows;
    }
    const int r0 = warp * RPW; // first tile row of this warp
    const std::int64_t row0 = row_begin + static_cast<std::int64_t>(t) * p.tile_rows;

    // the lane that will write result `value_index` fetches its bias now, behind the math
    const int value_index = (lane * kV) >> 5; // = r * MT + mi
    const bool writer_lane = (lane & (32 / kV - 1)) == 0;
    const int out_r = r0 + value_index / MT;
    const int out_m = m_base + value_index % MT;
    const bool out_valid = writer_lane && out_r < rows && out_m < p.m_total;
    float bias = 0.0f;
    if (out_valid && p.w.bias != nullptr) {
      bias = __ldg(p.w.bias + row0 + out_r);
    }

    if (!ptx::MbarWait(&full_bar[s], round & 1u)) {
      ReportStatus(p.status, kDeviceTimeoutFullBarrier);
      return;
    }
    const unsigned char *sb = stage_base + static_cast<size_t>(s) * p.stage_bytes;
    const float *ss = reinterpret_cast<const float *>(sb + p.stage_b_bytes);
    const unsigned char *sz = sb + p.stage_b_bytes + p.stage_scale_bytes;

    float acc[kV];
#pragma unroll
    for (int v = 0; v < kV; ++v) {
      acc[v] = 0.0f;
    }
    if (r0 < rows) {
      // Rows of this warp that lie beyond the tile read the warp's first row instead (their
      // sums are never written), which keeps the row loop free of branches so that the
      // independent rows interleave in the instruction stream.
      int row_of[RPW];
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        row_of[r] = r0 + r < rows ? r0 + r : r0;
      }
#ifndef MNB_GEMV_SKIP_COMPUTE
#pragma unroll 1
      for (int j = 0; j < p.chunk_iters; ++j) {
        const int c = lane + 32 * j;
        const int c_read = c < p.chunks_per_row ? c : 0; // padded chunk columns have zero activations
        const int block = (c_read * kW) >> p.block_shift;
        std::uint64_t ap[MT][Traits::kPairs];
        float a_sum[MT];
#pragma unroll
        for (int mi = 0; mi < MT; ++mi) {
          const unsigned char *arow = act_base + mi * act_m_bytes;
#pragma unroll
          for (int u = 0; u < Traits::kUnits; ++u) {
            const uint4 v = *reinterpret_cast<const uint4 *>(arow + ActUnitOffset(c * Traits::kUnits + u));
            asm("mov.b64 %0, {%1, %2};" : "=l"(ap[mi][2 * u]) : "r"(v.x), "r"(v.y));
            asm("mov.b64 %0, {%1, %2};" : "=l"(ap[mi][2 * u + 1]) : "r"(v.z), "r"(v.w));
          }
          a_sum[mi] = reinterpret_cast<const float *>(arow + act_row_bytes)[c];
        }
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          const int row = row_of[r];
          const uint4 q = *reinterpret_cast<const uint4 *>(sb + static_cast<size_t>(row) * p.w.row_bytes +
                                                           static_cast<size_t>(c_read) * kChunkBytes);
          const float scale = ss[row * p.w.n_blocks + block];
          int zp = default_zp;
          if (has_zp) {
            if constexpr (BITS == 8) {
              zp = sz[row * p.w.zp_row_bytes + block];
            } else {
              const int byte = sz[row * p.w.zp_row_bytes + (block >> 1)];
              zp = (byte >> ((block & 1) * 4)) & 0x0f;
            }
          }
          const float neg_zp = -static_cast<float>(zp);
#pragma unroll
          for (int mi = 0; mi < MT; ++mi) {
            const float raw = ChunkDot<BITS>(q, ap[mi], magic, neg_magic2);
            acc[r * MT + mi] = fmaf(scale, fmaf(neg_zp, a_sum[mi], raw), acc[r * MT + mi]);
          }
        }
      }
#endif
    }
    // this warp is done with the stage
    __syncwarp();
    if (lane == 0) {
      ptx::MbarArrive(&empty_bar[s]);
    }
    const float mine = WarpMultiReduce<kV>(acc, lane);
    if (out_valid) {
      p.out.y[static_cast<std::int64_t>(out_m) * p.out.ld + p.out.col_offset + row0 + out_r] = mine + bias;
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

// ------------------------------------------------------------------------------------------
// Word-wise kernels for the shapes no staged kernel takes (block_size 16, 8-bit rows too long for
// whole-row stages, row sizes outside the chunked layouts). The unit is a group of eight consecutive
// codes, 4 bytes of a 4-bit row or 8 of an 8-bit one, read straight from global memory, so every
// weight byte is read once per pass of MT tokens. A group never straddles a quantization block
// (block_size >= 16). Arithmetic: codes as exact floats, fp32 FMAs.
template <int BITS> struct GroupWord;
template <> struct GroupWord<4> {
  using Type = std::uint32_t;
};
template <> struct GroupWord<8> {
  using Type = uint2;
};

// The eight codes of a group minus the block's zero point, as floats: 2^23 + code assembled in the
// mantissa, minus (2^23 + zp), which is exact and needs no integer-to-float conversion. `magic` (the
// bits of 2^23) arrives as a kernel argument: with the constant visible the compiler turns the pair
// back into conversions, which run at a fraction of the FMA rate (55 % of the conversion pipe, and
// that the limit, on an 8-bit M = 1 node). `neg_offset` = -(2^23 + zp) = -as_float(magic | zp).
template <int BITS>
__device__ __forceinline__ void DecodeEightCodes(typename GroupWord<BITS>::Type q, std::uint32_t magic,
                                                 float neg_offset, float (&code)[8]) {
  if constexpr (BITS == 4) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      code[e] = __uint_as_float(((q >> (4 * e)) & 0x0fu) | magic) + neg_offset;
    }
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      code[e] = __uint_as_float(((q.x >> (8 * e)) & 0xffu) | magic) + neg_offset;
      code[4 + e] = __uint_as_float(((q.y >> (8 * e)) & 0xffu) | magic) + neg_offset;
    }
  }
}

// Eight activations of token row `src` from column k0 on; zeros beyond K (padding codes meet zeros).
__device__ __forceinline__ void LoadEightActivations(const float *src, int k0, int k, bool vector, float (&av)[8]) {
  if (vector && k0 + 8 <= k) {
    const float4 lo = __ldg(reinterpret_cast<const float4 *>(src + k0));
    const float4 hi = __ldg(reinterpret_cast<const float4 *>(src + k0) + 1);
    av[0] = lo.x, av[1] = lo.y, av[2] = lo.z, av[3] = lo.w;
    av[4] = hi.x, av[5] = hi.y, av[6] = hi.z, av[7] = hi.w;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      av[e] = k0 + e < k ? __ldg(src + k0 + e) : 0.0f;
    }
  }
}

// One and two tokens: one warp per output column, lanes stride over the groups of the row (the
// loads of a warp are contiguous), four groups per lane at a time with the words of the next four
// requested before these are used. acc += scale * sum a * (code - zp).
template <int BITS, int MT>
__global__ void __launch_bounds__(256)
    nbits_gemv_words_kernel(const WeightView w, const float *a, int m_total, OutputView out, int block_shift,
                            int a_vector, std::uint32_t magic) {
  using Word = typename GroupWord<BITS>::Type;
  constexpr int kBatch = 4;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const std::int64_t col = static_cast<std::int64_t>(blockIdx.x) * 8 + warp;
  const int m_base = blockIdx.y * MT;
  if (col >= w.n) {
    return;
  }
  float acc[MT];
#pragma unroll
  for (int mi = 0; mi < MT; ++mi) {
    acc[mi] = 0.0f;
  }
  const Word *row = reinterpret_cast<const Word *>(w.b + col * w.row_bytes);
  const float *scales = w.scales + col * w.n_blocks;
  const std::uint8_t *zero_points = w.zp != nullptr ? w.zp + col * w.zp_row_bytes : nullptr;
  const float *token[MT];
#pragma unroll
  for (int mi = 0; mi < MT; ++mi) {
    // a token beyond M repeats the last one; its sum is not written
    token[mi] = a + static_cast<std::int64_t>(m_base + mi < m_total ? m_base + mi : m_total - 1) * w.k;
  }
  const int k = static_cast<int>(w.k);
  const int groups = (k + 7) / 8; // groups with at least one code below K
  const bool vector = a_vector != 0;

  auto consume = [&](int g, Word q) {
    const int k0 = g * 8;
    const int block = k0 >> block_shift;
    std::uint32_t zp = 1u << (BITS - 1);
    if (zero_points != nullptr) {
      if constexpr (BITS == 8) {
        zp = __ldg(zero_points + block);
      } else {
        zp = (__ldg(zero_points + (block >> 1)) >> ((block & 1) * 4)) & 0x0fu;
      }
    }
    const float scale = __ldg(scales + block);
    float code[8];
    DecodeEightCodes<BITS>(q, magic, -__uint_as_float(magic | zp), code);
#pragma unroll
    for (int mi = 0; mi < MT; ++mi) {
      float av[8];
      LoadEightActivations(token[mi], k0, k, vector, av);
      float even = av[0] * code[0];
      float odd = av[1] * code[1];
#pragma unroll
      for (int e = 2; e < 8; e += 2) {
        even = fmaf(av[e], code[e], even);
        odd = fmaf(av[e + 1], code[e + 1], odd);
      }
      acc[mi] = fmaf(scale, even + odd, acc[mi]);
    }
  };

  // batches of four groups per lane; the words of the next batch are requested before this one is used
  const int batches = groups / (32 * kBatch);
  Word ahead[kBatch];
  if (batches > 0) {
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      ahead[u] = __ldg(row + lane + 32 * u);
    }
  }
#pragma unroll 1
  for (int batch = 0; batch < batches; ++batch) {
    const int g = batch * 32 * kBatch + lane;
    Word now[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      now[u] = ahead[u];
    }
    if (batch + 1 < batches) {
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        ahead[u] = __ldg(row + g + 32 * (kBatch + u));
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      consume(g + 32 * u, now[u]);
    }
  }
  for (int g = batches * 32 * kBatch + lane; g < groups; g += 32) {
    consume(g, __ldg(row + g));
  }
#pragma unroll
  for (int mi = 0; mi < MT; ++mi) {
    float v = acc[mi];
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      v += __shfl_xor_sync(0xffffffffu, v, offset);
    }
    if (lane == 0 && m_base + mi < m_total) {
      const float bias = w.bias != nullptr ? __ldg(w.bias + col) : 0.0f;
      out.y[static_cast<std::int64_t>(m_base + mi) * out.ld + out.col_offset + col] = v + bias;
    }
  }
}

// Three and more tokens: a lane per output column, so that the activations of a group are one
// address for the whole warp (with lanes along K every lane loads its own eight activations per
// token: one load per FMA). A CTA takes 32 columns; its eight warps take alternate chunks of 16
// groups (128 codes) of K. Per chunk a warp copies into a tile of shared memory of its own, with
// loads that run along K: the words of its 32 columns, their scales and zero points, and the
// chunk's activations of up to eight tokens. It then reads the words back one column per lane and
// the activations as broadcast loads, four tokens at a time so that four dot products are in
// flight. The partial sums of the warps meet in shared memory at the end. No CTA-wide barrier in
// the loop.
constexpr int kColumnsWarps = 8;      // sixteen when the node has no more 32-column CTAs than the GPU has SMs
constexpr int kColumnsChunk = 16;      // groups per chunk
constexpr int kColumnsWordStride = 17; // words of a column in the tile, padded
constexpr int kColumnsMetaStride = 9;  // up to 8 blocks per chunk (block_size 16), padded
constexpr int kColumnsTokens = 8;      // tokens per pass

template <int BITS> __host__ __device__ constexpr int ColumnsWordBytes() { return 32 * kColumnsWordStride * BITS; }
constexpr int kColumnsMetaBytes = 32 * kColumnsMetaStride * 8;
template <int BITS, int MT> __host__ __device__ constexpr int ColumnsWarpBytes() {
  return ColumnsWordBytes<BITS>() + kColumnsMetaBytes + MT * kColumnsChunk * 8 * 4;
}

template <int BITS, int MT>
__global__ void __launch_bounds__(2 * kColumnsWarps * 32)
    nbits_gemv_columns_kernel(const WeightView w, const float *a, int m_total, OutputView out, int block_shift,
                              int a_vector, std::uint32_t magic) {
  static_assert(MT % 4 == 0, "tokens are taken four at a time");
  using Word = typename GroupWord<BITS>::Type;
  extern __shared__ __align__(16) unsigned char columns_smem[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const std::int64_t col0 = static_cast<std::int64_t>(blockIdx.x) * 32;
  const int m_base = blockIdx.y * MT;
  const int tokens = m_total - m_base < MT ? m_total - m_base : MT;
  const int warps = static_cast<int>(blockDim.x >> 5);
  unsigned char *mine = columns_smem + warp * ColumnsWarpBytes<BITS, MT>();
  Word *words = reinterpret_cast<Word *>(mine);
  float2 *meta = reinterpret_cast<float2 *>(mine + ColumnsWordBytes<BITS>());
  float *acts = reinterpret_cast<float *>(mine + ColumnsWordBytes<BITS>() + kColumnsMetaBytes); // [MT][128]

  float acc[MT];
#pragma unroll
  for (int mi = 0; mi < MT; ++mi) {
    acc[mi] = 0.0f;
  }
  constexpr int kChunkCodes = kColumnsChunk * 8;
  const int groups = static_cast<int>((w.k + 7) / 8);
  const int chunks = (groups + kColumnsChunk - 1) / kColumnsChunk;
  // quantization blocks a chunk touches (one for block_size >= 128)
  const int blocks_per_chunk = (kChunkCodes >> block_shift) > 0 ? (kChunkCodes >> block_shift) : 1;
  const int columns_here = w.n - col0 < 32 ? static_cast<int>(w.n - col0) : 32;

  for (int chunk = warp; chunk < chunks; chunk += warps) {
    const int g0 = chunk * kColumnsChunk;
    const std::int64_t k_first = static_cast<std::int64_t>(g0) * 8;
    const int first_block = static_cast<int>(k_first >> block_shift);
    __syncwarp(); // the tiles of the chunk before have been read
    // words: two columns per step, sixteen lanes along K each; columns beyond N repeat the last one
    {
      const int gl = lane & 15;
#pragma unroll 8
      for (int step = 0; step < 16; ++step) {
        const int c = 2 * step + (lane >> 4);
        const std::int64_t col = col0 + (c < columns_here ? c : columns_here - 1);
        Word q{};
        if (g0 + gl < groups) {
          q = __ldg(reinterpret_cast<const Word *>(w.b + col * w.row_bytes) + g0 + gl);
        }
        words[c * kColumnsWordStride + gl] = q;
      }
    }
    // {scale, -(2^23 + zp)} of every (column, block of the chunk)
    for (int item = lane; item < 32 * blocks_per_chunk; item += 32) {
      const int c = item / blocks_per_chunk;
      const int b = item - c * blocks_per_chunk;
      const std::int64_t col = col0 + (c < columns_here ? c : columns_here - 1);
      const int block = first_block + b;
      if (block < w.n_blocks) {
        meta[c * kColumnsMetaStride + b] =
            make_float2(__ldg(w.scales + col * w.n_blocks + block),
                        -__uint_as_float(magic | static_cast<std::uint32_t>(ZeroPointOf(w, col, block))));
      }
    }
    // activations of the chunk: 128 per token, four per lane; zeros beyond K and beyond M
#pragma unroll
    for (int mi = 0; mi < MT; ++mi) {
      const std::int64_t kk = k_first + 4 * lane;
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (mi < tokens) {
        const float *src = a + static_cast<std::int64_t>(m_base + mi) * w.k;
        if (a_vector != 0 && kk + 4 <= w.k) {
          v = __ldg(reinterpret_cast<const float4 *>(src + kk));
        } else {
          v.x = kk + 0 < w.k ? __ldg(src + kk + 0) : 0.0f;
          v.y = kk + 1 < w.k ? __ldg(src + kk + 1) : 0.0f;
          v.z = kk + 2 < w.k ? __ldg(src + kk + 2) : 0.0f;
          v.w = kk + 3 < w.k ? __ldg(src + kk + 3) : 0.0f;
        }
      }
      reinterpret_cast<float4 *>(acts + mi * kChunkCodes)[lane] = v;
    }
    __syncwarp();
    const int here = groups - g0 < kColumnsChunk ? groups - g0 : kColumnsChunk;
#pragma unroll 2
    for (int gi = 0; gi < here; ++gi) {
      const int block = static_cast<int>((k_first + gi * 8) >> block_shift) - first_block;
      const float2 sz = meta[lane * kColumnsMetaStride + block];
      float code[8]; // code - zp: small integers, exact
      DecodeEightCodes<BITS>(words[lane * kColumnsWordStride + gi], magic, sz.y, code);
#pragma unroll
      for (int quad = 0; quad < MT; quad += 4) {
        float4 lo[4];
        float4 hi[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float4 *src = reinterpret_cast<const float4 *>(acts + (quad + t) * kChunkCodes + gi * 8);
          lo[t] = src[0];
          hi[t] = src[1];
        }
        float dot[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          dot[t] = lo[t].x * code[0];
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          dot[t] = fmaf(lo[t].y, code[1], dot[t]);
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          dot[t] = fmaf(lo[t].z, code[2], dot[t]);
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          dot[t] = fmaf(lo[t].w, code[3], dot[t]);
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          dot[t] = fmaf(hi[t].x, code[4], dot[t]);
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          dot[t] = fmaf(hi[t].y, code[5], dot[t]);
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          dot[t] = fmaf(hi[t].z, code[6], dot[t]);
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          dot[t] = fmaf(hi[t].w, code[7], dot[t]);
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          acc[quad + t] = fmaf(sz.x, dot[t], acc[quad + t]);
        }
      }
    }
  }
  // sum over the warps: [warp][token][column] in the shared memory the tiles used
  __syncthreads();
  float *partial = reinterpret_cast<float *>(columns_smem);
#pragma unroll
  for (int mi = 0; mi < MT; ++mi) {
    partial[(warp * MT + mi) * 32 + lane] = acc[mi];
  }
  __syncthreads();
  for (int item = threadIdx.x; item < tokens * 32; item += warps * 32) {
    const int mi = item >> 5;
    const int c = item & 31;
    if (c < columns_here) {
      float total = 0.0f;
      for (int wi = 0; wi < warps; ++wi) {
        total += partial[(wi * MT + mi) * 32 + c];
      }
      const float bias = w.bias != nullptr ? __ldg(w.bias + col0 + c) : 0.0f;
      out.y[static_cast<std::int64_t>(m_base + mi) * out.ld + out.col_offset + col0 + c] = total + bias;
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

template <int BITS, int MT, int RPW>
cudaError_t LaunchStreamInstance(const StreamParams &p, dim3 grid, size_t smem, cudaStream_t stream) {
  auto kernel = nbits_gemv_stream_kernel<BITS, MT, RPW>;
  // per device and cheap: set on every launch rather than caching across devices
  const cudaError_t attr =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (attr != cudaSuccess) {
    return attr;
  }
  kernel<<<grid, kThreads, smem, stream>>>(p);
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
  const int mt = m == 1 ? 1 : 2;
  StreamParams p{};
  p.w = w;
  p.a = a;
  p.m_total = static_cast<int>(m);
  p.out = out;
  p.status = status_word;
  p.magic = kMagicBits;
  p.chunks_per_row = w.row_bytes / kChunkBytes;
  p.chunk_iters = (p.chunks_per_row + 31) / 32;
  p.block_shift = Log2Exact(w.block_size);
  const int units_per_chunk = w.bits == 4 ? 8 : 4;
  const int chunk_slots = p.chunk_iters * 32;
  p.a_bytes = mt * (chunk_slots * units_per_chunk * 16 + chunk_slots * 4);
  p.a_bytes = (p.a_bytes + 127) & ~127;
  const size_t barrier_bytes = 2 * kMaxStages * sizeof(std::uint64_t);
  const size_t budget = 226 * 1024 - barrier_bytes - static_cast<size_t>(p.a_bytes);
  if (static_cast<size_t>(p.a_bytes) + barrier_bytes + 32 * 1024 > 226 * 1024) {
    return nullptr; // K too large to keep the activations in shared memory
  }
  int rpw = 4;
  for (;; rpw >>= 1) {
    p.rows_per_warp = rpw;
    p.tile_rows = kConsumerWarps * rpw;
    p.stage_b_bytes = p.tile_rows * w.row_bytes;
    p.stage_scale_bytes = (p.tile_rows * w.n_blocks * 4 + 15) & ~15;
    p.stage_zp_bytes = w.zp != nullptr ? ((p.tile_rows * w.zp_row_bytes + 15) & ~15) : 0;
    p.stage_bytes = (p.stage_b_bytes + p.stage_scale_bytes + p.stage_zp_bytes + 127) & ~127;
    p.stages = static_cast<int>(budget / static_cast<size_t>(p.stage_bytes));
    if (p.stages > kMaxStages) {
      p.stages = kMaxStages;
    }
    if (p.stages >= 2 || rpw == 1) {
      break;
    }
  }
  if (p.stages < 2) {
    return nullptr;
  }
  const size_t smem = static_cast<size_t>(p.stages) * p.stage_bytes + p.a_bytes + barrier_bytes;

  int ctas = sm_count > 0 ? sm_count : 148;
  // hand out rows in multiples of rows_per_warp so that warps stay fully used
  const std::int64_t groups = (w.n + rpw - 1) / rpw;
  if (ctas > groups) {
    ctas = static_cast<int>(groups);
  }
  p.rows_per_cta = static_cast<int>((groups + ctas - 1) / ctas) * rpw;

  dim3 grid(static_cast<unsigned>(ctas), static_cast<unsigned>((m + mt - 1) / mt), 1);
  cudaError_t err = cudaErrorInvalidValue;
  const char *name = nullptr;
#define MNB_STREAM_CASE(B_, M_, R_)                                                              \
  if (w.bits == B_ && mt == M_ && rpw == R_) {                                                   \
    err = LaunchStreamInstance<B_, M_, R_>(p, grid, smem, stream);                               \
    name = "nbits_gemv_stream_kernel<" #B_ "," #M_ "," #R_ ">";                                  \
  }
  MNB_STREAM_CASE(4, 1, 4)
  MNB_STREAM_CASE(4, 1, 2)
  MNB_STREAM_CASE(4, 1, 1)
  MNB_STREAM_CASE(4, 2, 4)
  MNB_STREAM_CASE(4, 2, 2)
  MNB_STREAM_CASE(4, 2, 1)
  MNB_STREAM_CASE(8, 1, 4)
  MNB_STREAM_CASE(8, 1, 2)
  MNB_STREAM_CASE(8, 1, 1)
  MNB_STREAM_CASE(8, 2, 4)
  MNB_STREAM_CASE(8, 2, 2)
  MNB_STREAM_CASE(8, 2, 1)
#undef MNB_STREAM_CASE
  if (err != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return name;
}

namespace {

template <int BITS, int MT>
cudaError_t LaunchWordsInstance(const WeightView &w, const float *a, std::int64_t m, OutputView out, int a_vector,
                                cudaStream_t stream) {
  dim3 grid(static_cast<unsigned>((w.n + 7) / 8), static_cast<unsigned>((m + MT - 1) / MT), 1);
  nbits_gemv_words_kernel<BITS, MT>
      <<<grid, 256, 0, stream>>>(w, a, static_cast<int>(m), out, Log2Exact(w.block_size), a_vector, kMagicBits);
  return cudaGetLastError();
}

template <int BITS, int MT>
cudaError_t LaunchColumnsInstance(const WeightView &w, const float *a, std::int64_t m, OutputView out, int a_vector,
                                  cudaStream_t stream, int sm_count) {
  auto kernel = nbits_gemv_columns_kernel<BITS, MT>;
  static_assert(ColumnsWarpBytes<BITS, MT>() >= MT * 32 * 4, "the partial sums reuse the tiles");
  dim3 grid(static_cast<unsigned>((w.n + 31) / 32), static_cast<unsigned>((m + MT - 1) / MT), 1);
  // a narrow node in one pass leaves SMs with one CTA or none: twice the warps along K then
  const int warps = static_cast<std::int64_t>(grid.x) * grid.y <= (sm_count > 0 ? sm_count : 148) ? 2 * kColumnsWarps
                                                                                                  : kColumnsWarps;
  const int smem = warps * ColumnsWarpBytes<BITS, MT>();
  const cudaError_t attr =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * kColumnsWarps * ColumnsWarpBytes<BITS, MT>());
  if (attr != cudaSuccess) {
    return attr;
  }
  kernel<<<grid, warps * 32, smem, stream>>>(w, a, static_cast<int>(m), out, Log2Exact(w.block_size),
                                                      a_vector, kMagicBits);
  return cudaGetLastError();
}

template <int BITS>
cudaError_t LaunchWordsBits(const WeightView &w, const float *a, std::int64_t m, OutputView out, int a_vector,
                            cudaStream_t stream, int sm_count, const char **name) {
  *name = "nbits_gemv_words_kernel";
  if (m == 1) {
    return LaunchWordsInstance<BITS, 1>(w, a, m, out, a_vector, stream);
  }
  if (m == 2) {
    return LaunchWordsInstance<BITS, 2>(w, a, m, out, a_vector, stream);
  }
  *name = "nbits_gemv_columns_kernel";
  if (m <= 4) {
    return LaunchColumnsInstance<BITS, 4>(w, a, m, out, a_vector, stream, sm_count);
  }
  return LaunchColumnsInstance<BITS, kColumnsTokens>(w, a, m, out, a_vector, stream, sm_count); // more tokens: passes of eight
}

} // namespace

const char *LaunchGemvWords(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                            cudaStream_t stream, int sm_count) {
  if (m < 1 || w.n < 1 || w.k < 1 || w.k > (std::int64_t{1} << 30) || (w.bits != 4 && w.bits != 8) ||
      w.block_size < 16) {
    return nullptr;
  }
  // a group of eight codes is one aligned 4-byte (4-bit) or 8-byte (8-bit) load
  const std::uintptr_t group_bytes = static_cast<std::uintptr_t>(w.bits);
  if ((reinterpret_cast<std::uintptr_t>(w.b) % group_bytes) != 0 || (w.row_bytes % group_bytes) != 0) {
    return nullptr;
  }
  const int a_vector = (w.k % 4) == 0 && (reinterpret_cast<std::uintptr_t>(a) & 15u) == 0 ? 1 : 0;
  const char *name = nullptr;
  const cudaError_t err = w.bits == 4 ? LaunchWordsBits<4>(w, a, m, out, a_vector, stream, sm_count, &name)
                                      : LaunchWordsBits<8>(w, a, m, out, a_vector, stream, sm_count, &name);
  if (err != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return name;
}

const char *LaunchGemvGeneric(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                              cudaStream_t stream, int sm_count) {
  if (m < 1 || w.n < 1) {
    return nullptr;
  }
  if (const char *words = LaunchGemvWords(w, a, m, out, stream, sm_count)) {
    return words;
  }
  cudaGetLastError();
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
