// Prefill path of MatMulNBits for sm_100a: dequantize-in-shared-memory GEMM on tcgen05/TMEM.
//
// Roles are swapped with respect to the textbook GEMM so that the packed weights never leave
// their natural [N, K] layout: the tensor core computes Y^T tiles,
//     D[n, m] = sum_k W[n, k] * A[m, k],
// with the dequantized weight tile as the MMA "A" operand (128 weight rows = 128 TMEM lanes)
// and an activation tile as the MMA "B" operand (BT tokens = BT TMEM columns).
//
// Per CTA (one output tile of 128 weight rows x BT tokens):
//   warp 0      TMA producer: per 64-wide k step, one 2-D tiled copy of the bf16 activation
//               tile (128-byte swizzle) and one of the packed weight tile (128 rows x 32 B)
//   warp 1      MMA issuer: one lane issues 4 tcgen05.mma (k = 16 each) per k step and commits
//               the stage's "empty" barrier; the last commit signals the accumulator
//   warps 2..9  dequantizers: read packed nibbles from shared memory, turn them into bf16
//               with a magic-number OR, subtract the zero point exactly, multiply by the
//               block scale, and store the 128-byte-swizzled K-major tile the MMA reads;
//               after the main loop the same warps are the epilogue: tcgen05.ld the fp32
//               accumulators, add bias, store Y (coalesced along n)
// Activations are converted fp32 -> bf16 (round to nearest even, the rounding of
// onnx_light_cpu/impl/math/half_conversion.h:80-87) by a pre-pass that also permutes k
// inside groups of eight to the order the nibble extraction produces.
// All barrier waits are bounded; on a timeout the CTA records a status word, skips to the
// tear-down, frees its TMEM columns and returns.

#include "nbits_common.cuh"
#include "nbits_ptx.cuh"
#include "nbits_tma.cuh"

#include <cuda_bf16.h>

#include <cstdint>

namespace mnb {
namespace {

constexpr int kTileN = 128;   // weight rows per CTA (UMMA M)
constexpr int kTileK = 64;    // k per pipeline stage (one 128-byte swizzle atom of bf16)
constexpr int kDequantWarps = 8;
constexpr int kThreads = (2 + kDequantWarps) * 32;

// Order in which the eight k of a group appear in the bf16 buffers: positions 0..7 hold
// k = 0,4,1,5,2,6,3,7. Extraction (w >> 4j) & 0x000F000F yields the pair (nibble j, nibble j+4).

__global__ void __launch_bounds__(256)
    nbits_a_to_bf16_kernel(const float *a, std::int64_t m, std::int64_t k, __nv_bfloat16 *out) {
  const std::int64_t groups_per_row = k / 8;
  const std::int64_t total = m * groups_per_row;
  for (std::int64_t g = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < total;
       g += static_cast<std::int64_t>(gridDim.x) * blockDim.x) {
    const float4 lo = __ldg(reinterpret_cast<const float4 *>(a) + 2 * g);
    const float4 hi = __ldg(reinterpret_cast<const float4 *>(a) + 2 * g + 1);
    // natural k: lo = (0,1,2,3), hi = (4,5,6,7); stored order 0,4,1,5,2,6,3,7
    __nv_bfloat162 p0 = __floats2bfloat162_rn(lo.x, hi.x);
    __nv_bfloat162 p1 = __floats2bfloat162_rn(lo.y, hi.y);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(lo.z, hi.z);
    __nv_bfloat162 p3 = __floats2bfloat162_rn(lo.w, hi.w);
    uint4 packed;
    packed.x = *reinterpret_cast<std::uint32_t *>(&p0);
    packed.y = *reinterpret_cast<std::uint32_t *>(&p1);
    packed.z = *reinterpret_cast<std::uint32_t *>(&p2);
    packed.w = *reinterpret_cast<std::uint32_t *>(&p3);
    reinterpret_cast<uint4 *>(out)[g] = packed;
  }
}

struct GemmParams {
  WeightView w;
  OutputView out;
  int m_total;
  int k_steps;
  int *status;
  int block_shift;
};

template <int BT> struct GemmSmem {
  static constexpr int kStageA = BT * 128;        // activation tile, bf16, swizzled
  static constexpr int kStageW = kTileN * 128;    // dequantized weight tile, bf16, swizzled
  static constexpr int kStageP = kTileN * 32;     // packed weight tile (4-bit: 32 B per row)
  static constexpr int kStage = kStageA + kStageW + kStageP;
  static constexpr int kStages = BT == 256 ? 4 : (BT == 128 ? 5 : 6);
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStage + kBarrierBytes + 1024; // + alignment slack
};

// Dequantizes 8 nibbles of `w` (one 16-byte output chunk in permuted k order).
__device__ __forceinline__ uint4 DequantWord(std::uint32_t w, __nv_bfloat162 offset,
                                             __nv_bfloat162 scale) {
  uint4 out;
  std::uint32_t v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const std::uint32_t bits = ((w >> (4 * j)) & 0x000f000fu) | 0x43004300u; // 128 + q, exact
    __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162 *>(&bits);
    x = __hsub2(x, offset);  // q - zp, exact
    x = __hmul2(x, scale);   // one bf16 rounding
    v[j] = *reinterpret_cast<std::uint32_t *>(&x);
  }
  out.x = v[0];
  out.y = v[1];
  out.z = v[2];
  out.w = v[3];
  return out;
}

template <int BT>
__global__ void __launch_bounds__(kThreads, 1)
    nbits_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                              const __grid_constant__ CUtensorMap map_p, const GemmParams p) {
  using Smem = GemmSmem<BT>;
  constexpr int kStages = Smem::kStages;
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms; the pointer stays in the
  // shared address space (no integer round trip) so that accesses compile to LDS/STS
  unsigned char *smem = smem_dyn + ((1024u - (ptx::SmemAddr(smem_dyn) & 1023u)) & 1023u);
  unsigned char *stage0 = smem;
  std::uint64_t *bars = reinterpret_cast<std::uint64_t *>(smem + kStages * Smem::kStage);
  std::uint64_t *full_tma = bars;               // [kStages] TMA landed
  std::uint64_t *full_deq = bars + kStages;     // [kStages] weights dequantized
  std::uint64_t *empty = bars + 2 * kStages;    // [kStages] MMAs of the stage retired
  std::uint64_t *accum_full = bars + 3 * kStages;
  std::uint32_t *tmem_slot = reinterpret_cast<std::uint32_t *>(bars + 3 * kStages + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n0 = blockIdx.x * kTileN;
  const int m0 = blockIdx.y * BT;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::MbarInit(&full_tma[s], 1);
      ptx::MbarInit(&full_deq[s], kDequantWarps);
      ptx::MbarInit(&empty[s], 1);
    }
    ptx::MbarInit(accum_full, 1);
    *abort_flag = 0;
    ptx::FenceMbarInit();
  }
  if (warp == 0) {
    ptx::TmemAlloc(tmem_slot, BT < 32 ? 32 : BT);
    ptx::TmemRelinquish();
  }
  ptx::TcFenceBefore();
  __syncthreads();
  ptx::TcFenceAfter();
  const std::uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      ptx::PrefetchTensorMap(&map_a);
      ptx::PrefetchTensorMap(&map_p);
      for (int ks = 0; ks < p.k_steps; ++ks) {
        const int s = ks % kStages;
        const std::uint32_t round = static_cast<std::uint32_t>(ks / kStages);
        if (!ptx::MbarWait(&empty[s], (round & 1u) ^ 1u)) {
          atomicExch(p.status, kDeviceTimeoutEmptyBarrier);
          *abort_flag = 1;
          break;
        }
        unsigned char *sa = stage0 + s * Smem::kStage;
        unsigned char *sp = sa + Smem::kStageA + Smem::kStageW;
        ptx::MbarArriveExpectTx(&full_tma[s], Smem::kStageA + Smem::kStageP);
        ptx::TmaLoad2D(sa, &map_a, ks * kTileK, m0, &full_tma[s]);
        ptx::TmaLoad2D(sp, &map_p, ks * (kTileK / 2), n0, &full_tma[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      constexpr std::uint32_t idesc = ptx::UmmaIdescBf16(kTileN, BT);
      bool ok = true;
      for (int ks = 0; ks < p.k_steps && ok; ++ks) {
        const int s = ks % kStages;
        const std::uint32_t round = static_cast<std::uint32_t>(ks / kStages);
        if (!ptx::MbarWait(&full_deq[s], round & 1u)) {
          atomicExch(p.status, kDeviceTimeoutMmaBarrier);
          *abort_flag = 1;
          ok = false;
          break;
        }
        ptx::TcFenceAfter();
        const std::uint32_t sa = ptx::SmemAddr(stage0 + s * Smem::kStage);
        const std::uint32_t sw = sa + Smem::kStageA;
#pragma unroll
        for (int kk = 0; kk < kTileK / 16; ++kk) {
          const std::uint64_t desc_w = ptx::UmmaDescKMajorSw128(sw + kk * 32);
          const std::uint64_t desc_a = ptx::UmmaDescKMajorSw128(sa + kk * 32);
          ptx::UmmaBf16(tmem_base, desc_w, desc_a, idesc, (ks | kk) != 0 ? 1u : 0u);
        }
        ptx::UmmaCommit(&empty[s]);
      }
      if (ok) {
        ptx::UmmaCommit(accum_full);
      }
    }
  } else {
    // ------------------------------- dequantizers -------------------------------
    const int dq = tid - 64;          // 0..255
    const int row = dq >> 1;          // weight row inside the tile
    const int half = dq & 1;          // which 32 of the 64 k of the stage
    const std::int64_t grow = static_cast<std::int64_t>(n0) + row;
    const bool row_valid = grow < p.w.n;
    const std::int64_t safe_row = row_valid ? grow : 0;
    const int default_zp = 8;

    auto load_meta = [&](int ks, float &scale, int &zp) {
      int block = (ks * kTileK + half * 32) >> p.block_shift;
      if (block >= p.w.n_blocks) {
        block = p.w.n_blocks - 1;
      }
      scale = row_valid ? __ldg(p.w.scales + safe_row * p.w.n_blocks + block) : 0.0f;
      zp = default_zp;
      if (p.w.zp != nullptr) {
        const int byte = __ldg(p.w.zp + safe_row * p.w.zp_row_bytes + (block >> 1));
        zp = (block & 1) ? (byte >> 4) : (byte & 0x0f);
      }
    };

    float scale_next;
    int zp_next;
    load_meta(0, scale_next, zp_next);
    bool ok = true;
    for (int ks = 0; ks < p.k_steps; ++ks) {
      const int s = ks % kStages;
      const std::uint32_t round = static_cast<std::uint32_t>(ks / kStages);
      const float scale = scale_next;
      const int zp = zp_next;
      if (ks + 1 < p.k_steps) {
        load_meta(ks + 1, scale_next, zp_next);
      }
      if (!ptx::MbarWait(&full_tma[s], round & 1u)) {
        atomicExch(p.status, kDeviceTimeoutFullBarrier);
        *abort_flag = 1;
        ok = false;
        break;
      }
      unsigned char *sa = stage0 + s * Smem::kStage;
      unsigned char *sw = sa + Smem::kStageA;
      const unsigned char *sp = sw + Smem::kStageW;
      const uint4 q = *reinterpret_cast<const uint4 *>(sp + row * 32 + half * 16);
      const __nv_bfloat162 offset = __float2bfloat162_rn(static_cast<float>(128 + zp));
      const __nv_bfloat162 scale2 = __float2bfloat162_rn(scale);
      const std::uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 chunk = DequantWord(words[i], offset, scale2);
        const int c = half * 4 + i; // 16-byte chunk index inside the 128-byte row
        *reinterpret_cast<uint4 *>(sw + row * 128 + ((c ^ (row & 7)) << 4)) = chunk;
      }
      // make the generic-proxy stores visible to the tensor core (async proxy), then signal
      ptx::FenceProxyAsyncShared();
      __syncwarp();
      if (lane == 0) {
        ptx::MbarArrive(&full_deq[s]);
      }
    }

    // ------------------------------- epilogue -------------------------------
    if (ok) {
      if (!ptx::MbarWait(accum_full, 0)) {
        atomicExch(p.status, kDeviceTimeoutEpilogueBarrier);
        *abort_flag = 1;
        ok = false;
      }
    }
    if (ok && *abort_flag == 0) {
      ptx::TcFenceAfter();
      const int quarter = warp & 3;            // TMEM lane quarter this warp may read
      const int col_half = (warp - 2) >> 2;    // two warps share a quarter: split the columns
      const int n_local = quarter * 32 + lane;
      const std::int64_t col = static_cast<std::int64_t>(n0) + n_local;
      const float bias = (p.w.bias != nullptr && col < p.w.n) ? __ldg(p.w.bias + col) : 0.0f;
      constexpr int kColsPerWarp = BT / 2;
#pragma unroll 1
      for (int c0 = 0; c0 < kColsPerWarp; c0 += 32) {
        const int tcol = col_half * kColsPerWarp + c0;
        std::uint32_t v[32];
        ptx::TmemLoad32x32(tmem_base + (static_cast<std::uint32_t>(quarter * 32) << 16) + tcol, v);
        ptx::TmemLoadWait();
        if (col < p.w.n) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = m0 + tcol + j;
            if (m < p.m_total) {
              p.out.y[static_cast<std::int64_t>(m) * p.out.ld + p.out.col_offset + col] =
                  __uint_as_float(v[j]) + bias;
            }
          }
        }
      }
    }
  }

  ptx::TcFenceBefore();
  __syncthreads();
  if (warp == 0) {
    ptx::TcFenceAfter();
    ptx::TmemDealloc(tmem_base, BT < 32 ? 32 : BT);
  }
}

// ---- host side -----------------------------------------------------------------------------

int Log2Of(int v) {
  int l = 0;
  while ((1 << l) < v) {
    ++l;
  }
  return l;
}

template <int BT>
const char *LaunchTile(const WeightView &w, std::int64_t m, const std::uint16_t *a_bf16,
                       OutputView out, int *status_word, cudaStream_t stream) {
  using Smem = GemmSmem<BT>;
  CUtensorMap map_a, map_p;
  if (!EncodeMap2D(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_bf16,
                   static_cast<std::uint64_t>(w.k), static_cast<std::uint64_t>(m),
                   static_cast<std::uint64_t>(w.k) * 2, kTileK, BT, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return nullptr;
  }
  if (!EncodeMap2D(&map_p, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w.b,
                   static_cast<std::uint64_t>(w.row_bytes), static_cast<std::uint64_t>(w.n),
                   static_cast<std::uint64_t>(w.row_bytes), kTileK / 2, kTileN,
                   CU_TENSOR_MAP_SWIZZLE_NONE)) {
    return nullptr;
  }
  GemmParams p{};
  p.w = w;
  p.out = out;
  p.m_total = static_cast<int>(m);
  p.k_steps = static_cast<int>(w.k / kTileK);
  p.status = status_word;
  p.block_shift = Log2Of(w.block_size);
  auto kernel = nbits_gemm_tcgen05_kernel<BT>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal) !=
      cudaSuccess) {
    return nullptr;
  }
  dim3 grid(static_cast<unsigned>((w.n + kTileN - 1) / kTileN),
            static_cast<unsigned>((m + BT - 1) / BT), 1);
  kernel<<<grid, kThreads, Smem::kTotal, stream>>>(map_a, map_p, p);
  if (cudaGetLastError() != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return BT == 256 ? "nbits_gemm_tcgen05_kernel<256>"
                   : (BT == 128 ? "nbits_gemm_tcgen05_kernel<128>" : "nbits_gemm_tcgen05_kernel<64>");
}

} // namespace

std::size_t GemmTcgen05ScratchBytes(std::int64_t m, std::int64_t k) {
  return static_cast<std::size_t>(m) * static_cast<std::size_t>(k) * 2;
}

bool GemmTcgen05Supports(const WeightView &w, std::int64_t m) {
  return m >= 1 && w.bits == 4 && w.block_size >= 32 && (w.k % kTileK) == 0 &&
         (reinterpret_cast<std::uintptr_t>(w.b) & 15u) == 0 && (w.row_bytes % 16) == 0 &&
         GetEncodeTiled() != nullptr;
}

const char *LaunchGemmTcgen05(const WeightView &w, const float *a, std::int64_t m,
                              std::uint16_t *a_bf16, OutputView out, int *status_word,
                              cudaStream_t stream, int sm_count) {
  if (!GemmTcgen05Supports(w, m) || (reinterpret_cast<std::uintptr_t>(a) & 15u) != 0) {
    return nullptr;
  }
  const std::int64_t groups = m * (w.k / 8);
  int blocks = static_cast<int>((groups + 255) / 256);
  const int max_blocks = (sm_count > 0 ? sm_count : 148) * 8;
  if (blocks > max_blocks) {
    blocks = max_blocks;
  }
  nbits_a_to_bf16_kernel<<<blocks, 256, 0, stream>>>(a, m, w.k,
                                                     reinterpret_cast<__nv_bfloat16 *>(a_bf16));
  if (cudaGetLastError() != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  const std::int64_t n_tiles = (w.n + kTileN - 1) / kTileN;
  const int sms = sm_count > 0 ? sm_count : 148;
  // pick the widest token tile that still gives every SM a tile
  if (m > 128 && n_tiles * ((m + 255) / 256) >= sms) {
    return LaunchTile<256>(w, m, a_bf16, out, status_word, stream);
  }
  if (m > 64) {
    return LaunchTile<128>(w, m, a_bf16, out, status_word, stream);
  }
  return LaunchTile<64>(w, m, a_bf16, out, status_word, stream);
}

} // namespace mnb
