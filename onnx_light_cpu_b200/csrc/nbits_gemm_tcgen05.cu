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
#include <cuda_fp16.h>

#include <cstdint>
#include <cstdlib>

namespace mnb {
namespace {

constexpr int kTileN = 128;   // weight rows per CTA (UMMA M)
constexpr int kTileK = 64;    // k per pipeline stage (one 128-byte swizzle atom of bf16)
constexpr int kDequantWarps = 8;
constexpr int kThreads = (2 + kDequantWarps) * 32;

// Order in which the eight k of a group appear in the bf16 buffers: positions 0..7 hold
// k = 0,4,1,5,2,6,3,7. Extraction (w >> 4j) & 0x000F000F yields the pair (nibble j, nibble j+4).

// `permute` = 0 keeps the natural order (8-bit codes are whole bytes and come out in order).
__global__ void __launch_bounds__(256)
    nbits_a_to_bf16_kernel(const float *a, std::int64_t m, std::int64_t k, __nv_bfloat16 *out, int permute) {
  // the GEMM behind this kernel may set itself up right away; its copies wait for this grid
  ptx::GridDependencyLaunch();
  // this kernel itself is launched behind whatever precedes it in the stream with programmatic
  // serialization (its blocks may be resident early): A and the scratch buffer are touched after that
  ptx::GridDependencyWait();
  const std::int64_t groups_per_row = k / 8;
  const std::int64_t total = m * groups_per_row;
  for (std::int64_t g = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < total;
       g += static_cast<std::int64_t>(gridDim.x) * blockDim.x) {
    const float4 lo = __ldg(reinterpret_cast<const float4 *>(a) + 2 * g);
    const float4 hi = __ldg(reinterpret_cast<const float4 *>(a) + 2 * g + 1);
    // natural k: lo = (0,1,2,3), hi = (4,5,6,7); stored order 0,4,1,5,2,6,3,7 when permuted
    __nv_bfloat162 p0 = permute != 0 ? __floats2bfloat162_rn(lo.x, hi.x) : __floats2bfloat162_rn(lo.x, lo.y);
    __nv_bfloat162 p1 = permute != 0 ? __floats2bfloat162_rn(lo.y, hi.y) : __floats2bfloat162_rn(lo.z, lo.w);
    __nv_bfloat162 p2 = permute != 0 ? __floats2bfloat162_rn(lo.z, hi.z) : __floats2bfloat162_rn(hi.x, hi.y);
    __nv_bfloat162 p3 = permute != 0 ? __floats2bfloat162_rn(lo.w, hi.w) : __floats2bfloat162_rn(hi.z, hi.w);
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
  std::uint32_t magic; // 0x43004300, passed at run time so that it stays in a register
  float *partial;      // split-K: [parts][m_total][n] partial products, summed by a kernel behind this one
};

template <int BT, int BITS> struct GemmSmem {
  static constexpr int kRowP = kTileK * BITS / 8; // packed bytes of a row per stage: 32 (4-bit) or 64 (8-bit)
  static constexpr int kStageA = BT * 128;        // activation tile, bf16, swizzled
  static constexpr int kStageW = kTileN * 128;    // dequantized weight tile, bf16, swizzled
  static constexpr int kStageP = kTileN * kRowP;  // packed weight tile
  static constexpr int kStage = kStageA + kStageW + kStageP;
  static constexpr int kStages = BT == 256 ? 4 : (BT == 128 ? 5 : 6);
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStage + kBarrierBytes + 1024; // + alignment slack
};

// Dequantizes the 8 nibbles of `w` into one 16-byte chunk of bf16 in the k order 0,4,1,5,2,6,3,7
// and stores it at shared address `dst`. One asm block so that the four results are born in the
// register quad the vector store needs. `magic` = 0x43004300 (128.0 twice), `offset` =
// (128 + zp) twice, `scale` = block scale twice.
__device__ __forceinline__ void DequantStore(std::uint32_t dst, std::uint32_t w, std::uint32_t magic,
                                             std::uint32_t offset, std::uint32_t scale) {
  asm volatile("{\n\t"
               ".reg .b32 x0, x1, x2, x3, s1, s2, s3;\n\t"
               "shr.u32 s1, %1, 4;\n\t"
               "shr.u32 s2, %1, 8;\n\t"
               "shr.u32 s3, %1, 12;\n\t"
               "lop3.b32 x0, %1, 0x000f000f, %2, 0xEA;\n\t"
               "lop3.b32 x1, s1, 0x000f000f, %2, 0xEA;\n\t"
               "lop3.b32 x2, s2, 0x000f000f, %2, 0xEA;\n\t"
               "lop3.b32 x3, s3, 0x000f000f, %2, 0xEA;\n\t"
               "sub.rn.bf16x2 x0, x0, %3;\n\t"
               "sub.rn.bf16x2 x1, x1, %3;\n\t"
               "sub.rn.bf16x2 x2, x2, %3;\n\t"
               "sub.rn.bf16x2 x3, x3, %3;\n\t"
               "mul.rn.bf16x2 x0, x0, %4;\n\t"
               "mul.rn.bf16x2 x1, x1, %4;\n\t"
               "mul.rn.bf16x2 x2, x2, %4;\n\t"
               "mul.rn.bf16x2 x3, x3, %4;\n\t"
               "st.shared.v4.b32 [%0], {x0, x1, x2, x3};\n\t"
               "}" ::"r"(dst),
               "r"(w), "r"(magic), "r"(offset), "r"(scale)
               : "memory");
}

// Eight 8-bit codes (two words, natural k order) into one 16-byte chunk of bf16: 1024 + q as fp16
// through a byte permute (0x6400 | q), minus 1024 + zp exactly, then (q - zp), an integer of at most
// eight significant bits and so exact in bf16, times the block scale in bf16: the same two
// roundings as the 4-bit form (scale to bf16, product to bf16).
__device__ __forceinline__ void DequantStore8(std::uint32_t dst, std::uint32_t w0, std::uint32_t w1,
                                              std::uint32_t offset16, std::uint32_t scale) {
  const __half2 off = *reinterpret_cast<const __half2 *>(&offset16);
  const __nv_bfloat162 sc = *reinterpret_cast<const __nv_bfloat162 *>(&scale);
  std::uint32_t x[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const std::uint32_t word = i < 2 ? w0 : w1;
    const std::uint32_t h = __byte_perm(word, 0x64646464u, (i & 1) ? 0x4342u : 0x4140u);
    const float2 f = __half22float2(__hsub2(*reinterpret_cast<const __half2 *>(&h), off));
    const __nv_bfloat162 v = __hmul2(__floats2bfloat162_rn(f.x, f.y), sc);
    x[i] = *reinterpret_cast<const std::uint32_t *>(&v);
  }
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3])
               : "memory");
}

// bf16 pair (v, v) from a float, round to nearest even.
__device__ __forceinline__ std::uint32_t Bf16Pair(float v) {
  std::uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %1;" : "=r"(d) : "f"(v));
  return d;
}

template <int BT, int BITS>
__global__ void __launch_bounds__(kThreads, 1)
    nbits_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                              const __grid_constant__ CUtensorMap map_p, const GemmParams p) {
  using Smem = GemmSmem<BT, BITS>;
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
  ptx::GridDependencyLaunch();   // what follows in the stream (the next call's pre-pass) may move in as SMs free up

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::MbarInit(&full_tma[s], 1);
      ptx::MbarInit(&full_deq[s], kDequantWarps / 2);   // the group of dequantizer warps that takes the step
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
      // the bf16 activations come from the pre-pass launched just before (programmatic dependent
      // launch): TMEM, barriers and descriptors are set up while it runs, the copies wait for it
      ptx::GridDependencyWait();
      for (int ks = 0; ks < p.k_steps; ++ks) {
        const int s = ks % kStages;
        const std::uint32_t round = static_cast<std::uint32_t>(ks / kStages);
        if (!ptx::MbarWaitHot(&empty[s], (round & 1u) ^ 1u)) {
          ReportStatus(p.status, kDeviceTimeoutEmptyBarrier);
          *abort_flag = 1;
          break;
        }
        unsigned char *sa = stage0 + s * Smem::kStage;
        unsigned char *sp = sa + Smem::kStageA + Smem::kStageW;
        ptx::MbarArriveExpectTx(&full_tma[s], Smem::kStageA + Smem::kStageP);
        ptx::TmaLoad2D(sa, &map_a, ks * kTileK, m0, &full_tma[s]);
        ptx::TmaLoad2D(sp, &map_p, ks * Smem::kRowP, n0, &full_tma[s]);
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
        if (!ptx::MbarWaitHot(&full_deq[s], round & 1u)) {
          ReportStatus(p.status, kDeviceTimeoutMmaBarrier);
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
    // Two groups of four warps take alternate k steps (a step's chain of wait, load, convert, store,
    // proxy fence and arrival is latency, not work: two of them run at any time); a thread converts
    // the same half of two rows 64 apart.
    const int dq = tid - 64;          // 0..255
    const int group = dq >> 7;
    const int gdq = dq & 127;
    const int row0 = gdq >> 1;        // rows row0 and row0 + 64 of the tile
    const int half = gdq & 1;         // which 32 of the 64 k of the stage
    const int last_block = p.w.n_blocks - 1;
    const std::uint32_t magic = p.magic;
    const float *scale_row[2];
    const std::uint8_t *zp_row[2];
    bool row_valid[2];
    int packed_offset[2];
    int store_base[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = row0 + i * 64;
      const std::int64_t grow = static_cast<std::int64_t>(n0) + row;
      row_valid[i] = grow < p.w.n;
      const std::int64_t safe_row = row_valid[i] ? grow : 0;
      scale_row[i] = p.w.scales + safe_row * p.w.n_blocks;
      zp_row[i] = p.w.zp != nullptr ? p.w.zp + safe_row * p.w.zp_row_bytes : nullptr;
      packed_offset[i] = Smem::kStageA + Smem::kStageW + row * Smem::kRowP + half * (Smem::kRowP / 2);
      store_base[i] = Smem::kStageA + row * 128;
    }
    int chunk_offset[4];              // 16-byte chunk c of a row sits at c ^ (row & 7); both rows agree in row & 7
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      chunk_offset[c] = ((half * 4 + c) ^ (row0 & 7)) << 4;
    }

    // Scale and zero point of a k step's block. The loads are issued one step of the group ahead and
    // nothing touches their results before that step begins (a conversion right behind the load
    // would expose the L2 latency in every step).
    auto block_of = [&](int ks) {
      const int block = (ks * kTileK + half * 32) >> p.block_shift;
      return block > last_block ? last_block : block;
    };
    auto fetch_meta = [&](int ks, float (&scale)[2], int (&zp_byte)[2]) {
      const int block = block_of(ks);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        scale[i] = row_valid[i] ? __ldg(scale_row[i] + block) : 0.0f;
        if constexpr (BITS == 4) {
          zp_byte[i] = zp_row[i] != nullptr ? __ldg(zp_row[i] + (block >> 1)) : 0x88;
        } else {
          zp_byte[i] = zp_row[i] != nullptr ? __ldg(zp_row[i] + block) : 128;
        }
      }
    };

    float scale_raw[2];
    int zp_raw[2];
    if (group < p.k_steps) {
      fetch_meta(group, scale_raw, zp_raw);
    }
    bool ok = true;
    for (int ks = group; ks < p.k_steps; ks += 2) {
      const int s = ks % kStages;
      const std::uint32_t phase = static_cast<std::uint32_t>(ks / kStages) & 1u;
      std::uint32_t scale2[2], offset2[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        scale2[i] = Bf16Pair(scale_raw[i]);
        if constexpr (BITS == 4) {
          const int zp = (zp_raw[i] >> ((block_of(ks) & 1) * 4)) & 0x0f;
          offset2[i] = Bf16Pair(static_cast<float>(128 + zp)); // exact in bf16
        } else {
          const __half2 both = __float2half2_rn(static_cast<float>(1024 + zp_raw[i])); // exact in fp16
          offset2[i] = *reinterpret_cast<const std::uint32_t *>(&both);
        }
      }
      if (ks + 2 < p.k_steps) {
        fetch_meta(ks + 2, scale_raw, zp_raw);
      }
      if (!ptx::MbarWaitHot(&full_tma[s], phase)) {
        ReportStatus(p.status, kDeviceTimeoutFullBarrier);
        *abort_flag = 1;
        ok = false;
        break;
      }
      unsigned char *stage = stage0 + s * Smem::kStage;
      const std::uint32_t base = ptx::SmemAddr(stage);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const std::uint32_t dst = base + store_base[i];
        if constexpr (BITS == 4) {
          const uint4 q = *reinterpret_cast<const uint4 *>(stage + packed_offset[i]);
          DequantStore(dst + chunk_offset[0], q.x, magic, offset2[i], scale2[i]);
          DequantStore(dst + chunk_offset[1], q.y, magic, offset2[i], scale2[i]);
          DequantStore(dst + chunk_offset[2], q.z, magic, offset2[i], scale2[i]);
          DequantStore(dst + chunk_offset[3], q.w, magic, offset2[i], scale2[i]);
        } else {
          const uint4 q0 = *reinterpret_cast<const uint4 *>(stage + packed_offset[i]);
          const uint4 q1 = *reinterpret_cast<const uint4 *>(stage + packed_offset[i] + 16);
          DequantStore8(dst + chunk_offset[0], q0.x, q0.y, offset2[i], scale2[i]);
          DequantStore8(dst + chunk_offset[1], q0.z, q0.w, offset2[i], scale2[i]);
          DequantStore8(dst + chunk_offset[2], q1.x, q1.y, offset2[i], scale2[i]);
          DequantStore8(dst + chunk_offset[3], q1.z, q1.w, offset2[i], scale2[i]);
        }
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
        ReportStatus(p.status, kDeviceTimeoutEpilogueBarrier);
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

// ---------------------------------------------------------------------------------------------
// CTA pairs: 512 weight rows x `tokens` (<= 256) per pair of SMs, for every product of more than
// sixteen tokens that is worth it (PairPlanFor below).
//
// Two CTAs of a cluster (the same pair of SMs) share every MMA (cta_group::2, 256 x tokens x 16): each
// CTA dequantizes 256 weight rows of its own (two 128-row sub-tiles = the two 256-column accumulators
// in its TMEM, all 512 columns) but stages only HALF of the token tile; the tensor cores of both SMs
// read both halves. Per 64-k step a CTA brings in at most 16 KB of activations and 8 KB of packed
// weights for 2 x 128 x 256 x 64 multiply-adds. The dequantized tile is transient, so it lives in
// buffers of its own instead of the TMA ring. (A single CTA with the whole 256-token tile, which this
// kernel replaced, was bound by shared-memory bandwidth: 176 KB crossed it per k step against 125 KB
// here, and 953 against 1076 TFLOP/s at M = 2048.)
//
// The dequantizers are bound by the latency of their own chain (wait, load, convert, store, proxy
// fence, arrive), so there are sixteen warps of them in two groups that take alternate k steps: two
// steps are being dequantized at any time. (Sixteen warps on every step: 1046 TFLOP/s; four groups
// with four buffers: 1066; five TMA stages: 1030; packed weights loaded from global memory by the
// dequantizers instead of TMA: 986.)
//
// Roles per CTA as in the 128-row kernel; the MMA issuer runs in the even CTA only. What crosses the pair:
//   w_full[b] of the even CTA collects the dequantizer warps of BOTH CTAs (the odd CTA's arrive
//     through the cluster address of that barrier). A warp arrives after it has seen its own CTA's
//     copies land, so one wait tells the issuer that weights and activations are in place in both.
//   empty[s], w_empty[b], accum_full are signalled in both CTAs by one tcgen05.commit.
// gridDim.z > 1 shares K between that many pairs per tile: each takes a consecutive part of the k
// steps and stores its partial tile, and nbits_split_k_sum_kernel behind this kernel adds the parts
// in order (+ bias), so the result does not depend on timing. (fp32 reductions straight into Y were
// tried first: 8.4 M element-wise L2 atomics took longer than the product.)
// TMEM is allocated and released by warp 0 of both CTAs together; a cluster barrier before the
// release keeps either CTA's shared memory and TMEM alive until both are done.

constexpr int kPairRows = 256;      // weight rows per CTA: two 128-row sub-tiles
constexpr int kPairTokens = 256;    // widest token tile of a pair = columns of one accumulator
constexpr int kPairDequantWarps = 16;
constexpr int kPairThreads = (2 + kPairDequantWarps) * 32;
constexpr int kPairGroups = 2;                                     // groups of dequantizer warps, one k step each
constexpr int kPairGroupThreads = kPairDequantWarps / kPairGroups * 32;
static_assert(kPairGroupThreads == 256, "a group covers 128 rows x two halves of a k step");
constexpr int kPairStages = 4;
constexpr int kPairBuffers = 3;
constexpr int kPairStageA = (kPairTokens / 2) * 128;   // half a token tile: 16 KB
constexpr int kPairBufW = kPairRows * 128;             // dequantized weights of a k step: 32 KB, two 16 KB sub-tiles
template <int BITS> struct PairSmem {
  static constexpr int kRowP = kTileK * BITS / 8;       // packed bytes of a row per k step: 32 (4-bit) or 64 (8-bit)
  static constexpr int kStageP = kPairRows * kRowP;     // packed weights of a k step: 8 or 16 KB
  static constexpr int kTotal = kPairStages * (kPairStageA + kStageP) + kPairBuffers * kPairBufW + 256 + 1024;
};

struct PairParams {
  GemmParams g;
  int tokens;       // token-tile width of the pair: a multiple of 16, <= 256
  std::uint32_t idesc;
};

template <int BITS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
    nbits_gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                                   const __grid_constant__ CUtensorMap map_p, const PairParams pp) {
  const GemmParams &p = pp.g;
  constexpr int kPairStageP = PairSmem<BITS>::kStageP;
  constexpr int kRowP = PairSmem<BITS>::kRowP;
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char *smem = smem_dyn + ((1024u - (ptx::SmemAddr(smem_dyn) & 1023u)) & 1023u);
  unsigned char *ring_a = smem;                                     // [stages][16 KB]
  unsigned char *buf_w = ring_a + kPairStages * kPairStageA;     // [buffers][32 KB]
  unsigned char *ring_p = buf_w + kPairBuffers * kPairBufW;         // [stages][8 KB]
  std::uint64_t *bars = reinterpret_cast<std::uint64_t *>(ring_p + kPairStages * kPairStageP);
  std::uint64_t *full_tma = bars;                    // [stages] this CTA's activations + packed weights landed
  std::uint64_t *empty = bars + kPairStages;         // [stages] pair MMAs that read the stage retired
  std::uint64_t *w_full = bars + 2 * kPairStages;    // [buffers] (even CTA) both CTAs' weights dequantized
  std::uint64_t *w_empty = w_full + kPairBuffers;    // [buffers] pair MMAs that read the buffer retired
  std::uint64_t *accum_full = w_empty + kPairBuffers;
  std::uint32_t *tmem_slot = reinterpret_cast<std::uint32_t *>(accum_full + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const std::uint32_t rank = ptx::ClusterCtaRank();      // 0: issues the MMAs
  ptx::GridDependencyLaunch();   // what follows in the stream (the sum of the parts, the next call's pre-pass) may move in as SMs free up
  const int n0 = blockIdx.x * kPairRows;                 // blockIdx.x = 2 * pair + rank
  const int m0 = blockIdx.y * pp.tokens;
  const int half_tokens = pp.tokens / 2;
  const std::uint32_t stage_a_bytes = static_cast<std::uint32_t>(half_tokens) * 128u;
  const int parts = static_cast<int>(gridDim.z);
  const int part = static_cast<int>(blockIdx.z);
  const int ks_begin = static_cast<int>(static_cast<std::int64_t>(part) * p.k_steps / parts);
  const int ks_end = static_cast<int>(static_cast<std::int64_t>(part + 1) * p.k_steps / parts);

  if (tid == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      ptx::MbarInit(&full_tma[s], 1);
      ptx::MbarInit(&empty[s], 1);
    }
    for (int b = 0; b < kPairBuffers; ++b) {
      ptx::MbarInit(&w_full[b], 2 * kPairDequantWarps / kPairGroups);
      ptx::MbarInit(&w_empty[b], 1);
    }
    ptx::MbarInit(accum_full, 1);
    *abort_flag = 0;
    ptx::FenceMbarInit();
  }
  if (warp == 0) {
    ptx::TmemAllocPair(tmem_slot, 512);
    ptx::TmemRelinquishPair();
  }
  ptx::TcFenceBefore();
  ptx::ClusterSync();   // barriers of both CTAs exist before anything arrives on them
  ptx::TcFenceAfter();
  const std::uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      ptx::PrefetchTensorMap(&map_a);
      ptx::PrefetchTensorMap(&map_p);
      ptx::GridDependencyWait();   // the bf16 activations come from the pre-pass launched just before
      int s = 0;
      std::uint32_t phase = 0;
      for (int ks = ks_begin; ks < ks_end; ++ks) {
        if (!ptx::MbarWaitHot(&empty[s], phase ^ 1u)) {
          ReportStatus(p.status, kDeviceTimeoutEmptyBarrier);
          *abort_flag = 1;
          break;
        }
        ptx::MbarArriveExpectTx(&full_tma[s], stage_a_bytes + kPairStageP);
        ptx::TmaLoad2D(ring_a + s * kPairStageA, &map_a, ks * kTileK, m0 + static_cast<int>(rank) * half_tokens,
                       &full_tma[s]);
        ptx::TmaLoad2D(ring_p + s * kPairStageP, &map_p, ks * kRowP, n0, &full_tma[s]);
        if (++s == kPairStages) {
          s = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (even CTA) -------------------------------
    if (lane == 0 && rank == 0) {
      bool ok = true;
      int s = 0;
      int b = 0;
      std::uint32_t b_phase = 0;
      for (int ks = ks_begin; ks < ks_end; ++ks) {
        if (!ptx::MbarWaitHot(&w_full[b], b_phase)) {
          ReportStatus(p.status, kDeviceTimeoutMmaBarrier);
          *abort_flag = 1;
          ok = false;
          break;
        }
        ptx::TcFenceAfter();
        const std::uint32_t sa = ptx::SmemAddr(ring_a + s * kPairStageA);
        const std::uint32_t sw = ptx::SmemAddr(buf_w + b * kPairBufW);
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
#pragma unroll
          for (int kk = 0; kk < kTileK / 16; ++kk) {
            const std::uint64_t desc_w = ptx::UmmaDescKMajorSw128(sw + sub * (kPairBufW / 2) + kk * 32);
            const std::uint64_t desc_a = ptx::UmmaDescKMajorSw128(sa + kk * 32);
            ptx::UmmaBf16Pair(tmem_base + sub * kPairTokens, desc_w, desc_a, pp.idesc, (ks != ks_begin || kk != 0) ? 1u : 0u);
          }
        }
        ptx::UmmaCommitPair(&empty[s], 3);
        ptx::UmmaCommitPair(&w_empty[b], 3);
        if (++s == kPairStages) {
          s = 0;
        }
        if (++b == kPairBuffers) {
          b = 0;
          b_phase ^= 1u;
        }
      }
      if (ok) {
        ptx::UmmaCommitPair(accum_full, 3);
      }
    }
  } else {
    // ------------------------------- dequantizers -------------------------------
    const int dq = tid - 64;                 // 0..511
    const int group = dq / kPairGroupThreads;  // takes k steps group, group + 2, ... of this CTA's part
    const int gdq = dq % kPairGroupThreads;
    const int row = gdq >> 1;                  // weight row inside each 128-row sub-tile
    const int half = gdq & 1;                  // which 32 of the 64 k of the stage
    const std::uint32_t magic = p.magic;
    const int last_block = p.w.n_blocks - 1;
    const float *scale_row[2];
    const std::uint8_t *zp_row[2];
    bool row_valid[2];
#pragma unroll
    for (int sub = 0; sub < 2; ++sub) {
      const std::int64_t grow = static_cast<std::int64_t>(n0) + sub * 128 + row;
      row_valid[sub] = grow < p.w.n;
      const std::int64_t safe_row = row_valid[sub] ? grow : 0;
      scale_row[sub] = p.w.scales + safe_row * p.w.n_blocks;
      zp_row[sub] = p.w.zp != nullptr ? p.w.zp + safe_row * p.w.zp_row_bytes : nullptr;
    }
    const int packed_offset = row * kRowP + half * (kRowP / 2);
    int store_offset[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = half * 4 + i; // 16-byte chunk index inside the 128-byte row
      store_offset[i] = row * 128 + ((c ^ (row & 7)) << 4);
    }
    // where this warp reports a dequantized buffer: the even CTA's barrier (the arrival form that
    // hands shared memory written by threads to the pair's MMA)
    const std::uint32_t w_full_even = ptx::MapToCta(ptx::SmemAddr(&w_full[0]), 0);

    // Scale and zero point of a k step's block: loaded one step of the group ahead, converted at the
    // start of the step that uses them (a conversion right behind the load would expose the L2 latency).
    auto block_of = [&](int ks) {
      const int block = (ks * kTileK + half * 32) >> p.block_shift;
      return block > last_block ? last_block : block;
    };
    auto fetch_meta = [&](int ks, float (&scale)[2], int (&zp_byte)[2]) {
      const int block = block_of(ks);
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        scale[sub] = row_valid[sub] ? __ldg(scale_row[sub] + block) : 0.0f;
        if constexpr (BITS == 4) {
          zp_byte[sub] = zp_row[sub] != nullptr ? __ldg(zp_row[sub] + (block >> 1)) : 0x88;
        } else {
          zp_byte[sub] = zp_row[sub] != nullptr ? __ldg(zp_row[sub] + block) : 128;
        }
      }
    };

    float scale_raw[2];
    int zp_raw[2];
    bool ok = true;
    int s = group;                // kPairGroups <= kPairStages, kPairBuffers
    std::uint32_t phase = 0;
    int b = group;
    std::uint32_t b_phase = 0;
    if (ks_begin + group < ks_end) {
      fetch_meta(ks_begin + group, scale_raw, zp_raw);
    }
    for (int ks = ks_begin + group; ks < ks_end; ks += kPairGroups) {
      [[maybe_unused]] const int shift = (block_of(ks) & 1) * 4;
      std::uint32_t scale2[2], offset2[2];
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        scale2[sub] = Bf16Pair(scale_raw[sub]);
        if constexpr (BITS == 4) {
          offset2[sub] = Bf16Pair(static_cast<float>(128 + ((zp_raw[sub] >> shift) & 0x0f))); // exact in bf16
        } else {
          const __half2 both = __float2half2_rn(static_cast<float>(1024 + zp_raw[sub])); // exact in fp16
          offset2[sub] = *reinterpret_cast<const std::uint32_t *>(&both);
        }
      }
      if (ks + kPairGroups < ks_end) {
        fetch_meta(ks + kPairGroups, scale_raw, zp_raw);
      }
      // this CTA's copies of the stage landed, and the buffer's previous readers have retired
      if (!ptx::MbarWaitHot(&full_tma[s], phase) || !ptx::MbarWaitHot(&w_empty[b], b_phase ^ 1u)) {
        ReportStatus(p.status, kDeviceTimeoutFullBarrier);
        *abort_flag = 1;
        ok = false;
        break;
      }
      const unsigned char *packed = ring_p + s * kPairStageP + packed_offset;
      unsigned char *dst = buf_w + b * kPairBufW;
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        const std::uint32_t tile = ptx::SmemAddr(dst + sub * (kPairBufW / 2));
        if constexpr (BITS == 4) {
          const uint4 q = *reinterpret_cast<const uint4 *>(packed + sub * 128 * kRowP);
          DequantStore(tile + store_offset[0], q.x, magic, offset2[sub], scale2[sub]);
          DequantStore(tile + store_offset[1], q.y, magic, offset2[sub], scale2[sub]);
          DequantStore(tile + store_offset[2], q.z, magic, offset2[sub], scale2[sub]);
          DequantStore(tile + store_offset[3], q.w, magic, offset2[sub], scale2[sub]);
        } else {
          const uint4 q0 = *reinterpret_cast<const uint4 *>(packed + sub * 128 * kRowP);
          const uint4 q1 = *reinterpret_cast<const uint4 *>(packed + sub * 128 * kRowP + 16);
          DequantStore8(tile + store_offset[0], q0.x, q0.y, offset2[sub], scale2[sub]);
          DequantStore8(tile + store_offset[1], q0.z, q0.w, offset2[sub], scale2[sub]);
          DequantStore8(tile + store_offset[2], q1.x, q1.y, offset2[sub], scale2[sub]);
          DequantStore8(tile + store_offset[3], q1.z, q1.w, offset2[sub], scale2[sub]);
        }
      }
      ptx::FenceProxyAsyncShared();
      __syncwarp();
      if (lane == 0) {
        ptx::MbarArriveCluster(w_full_even + static_cast<std::uint32_t>(b) * 8u);
      }
      s += kPairGroups;
      if (s >= kPairStages) {
        s -= kPairStages;
        phase ^= 1u;
      }
      b += kPairGroups;
      if (b >= kPairBuffers) {
        b -= kPairBuffers;
        b_phase ^= 1u;
      }
    }

    // ------------------------------- epilogue -------------------------------
    if (ok) {
      if (!ptx::MbarWait(accum_full, 0)) {
        ReportStatus(p.status, kDeviceTimeoutEpilogueBarrier);
        *abort_flag = 1;
        ok = false;
      }
    }
    if (ok && *abort_flag == 0) {
      ptx::TcFenceAfter();
      // four warps share a TMEM lane quarter: two accumulators x two halves of the token tile
      const int quarter = warp & 3;
      const int share = (warp - 2) >> 2;       // 0..3
      const int acc = share & 1;
      const int c_begin = (share >> 1) * (kPairTokens / 2);
      const int n_local = acc * 128 + quarter * 32 + lane;
      const std::int64_t col = static_cast<std::int64_t>(n0) + n_local;
      const bool whole = p.partial == nullptr;   // otherwise the sum kernel adds the bias
      const float bias = (whole && p.w.bias != nullptr && col < p.w.n) ? __ldg(p.w.bias + col) : 0.0f;
      float *part_out = whole ? nullptr : p.partial + static_cast<std::int64_t>(part) * p.m_total * p.w.n;
      const int m_end = (m0 + pp.tokens) < p.m_total ? (m0 + pp.tokens) : p.m_total;
#pragma unroll 1
      for (int c0 = c_begin; c0 < c_begin + kPairTokens / 2 && c0 < pp.tokens; c0 += 32) {
        std::uint32_t v[32];
        ptx::TmemLoad32x32(tmem_base + (static_cast<std::uint32_t>(quarter * 32) << 16) + acc * kPairTokens + c0, v);
        ptx::TmemLoadWait();
        if (col < p.w.n) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = m0 + c0 + j;
            if (m < m_end) {
              if (whole) {
                p.out.y[static_cast<std::int64_t>(m) * p.out.ld + p.out.col_offset + col] = __uint_as_float(v[j]) + bias;
              } else {
                part_out[static_cast<std::int64_t>(m) * p.w.n + col] = __uint_as_float(v[j]);
              }
            }
          }
        }
      }
    }
  }

  // both CTAs are done with each other's shared memory and with their TMEM
  __syncwarp();
  ptx::TcFenceBefore();
  ptx::ClusterSync();
  if (warp == 0) {
    ptx::TcFenceAfter();
    ptx::TmemDeallocPair(tmem_base, 512);
  }
}

// Y = part 0 + part 1 + ... (in that order) + bias, for a split-K product. The parts were written
// by the kernel before it and are still in L2.
__global__ void __launch_bounds__(256)
    nbits_split_k_sum_kernel(const float *partial, int parts, std::int64_t m, std::int64_t n, const float *bias,
                             OutputView out) {
  ptx::GridDependencyLaunch();
  ptx::GridDependencyWait();   // the partial products come from the kernel launched just before
  const std::int64_t total = m * n;
  for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += static_cast<std::int64_t>(gridDim.x) * 256) {
    const std::int64_t row = i / n;
    const std::int64_t col = i - row * n;
    float value = __ldcg(partial + i);
    for (int z = 1; z < parts; ++z) {
      value += __ldcg(partial + z * total + i);
    }
    out.y[row * out.ld + out.col_offset + col] = value + (bias != nullptr ? __ldg(bias + col) : 0.0f);
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

// Launch with programmatic stream serialization: the kernel's blocks may become resident while the
// kernel before it in the stream drains; it waits (griddepcontrol.wait) before it touches anything
// that kernel wrote.
template <typename Kernel, typename... Args>
bool LaunchDependent(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  if (cudaLaunchKernelEx(&config, kernel, args...) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return true;
}

// Launch with programmatic stream serialization behind the activation pre-pass.
template <typename Kernel>
bool LaunchBehindPrePass(Kernel kernel, dim3 grid, size_t smem, cudaStream_t stream, const CUtensorMap &map_a,
                         const CUtensorMap &map_p, const GemmParams &p) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  if (cudaLaunchKernelEx(&config, kernel, map_a, map_p, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return true;
}

template <int BT, int BITS>
const char *LaunchTileBits(const WeightView &w, std::int64_t m, const std::uint16_t *a_bf16,
                           OutputView out, int *status_word, cudaStream_t stream) {
  using Smem = GemmSmem<BT, BITS>;
  CUtensorMap map_a, map_p;
  if (!EncodeMap2D(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_bf16,
                   static_cast<std::uint64_t>(w.k), static_cast<std::uint64_t>(m),
                   static_cast<std::uint64_t>(w.k) * 2, kTileK, BT, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return nullptr;
  }
  if (!EncodeMap2D(&map_p, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w.b,
                   static_cast<std::uint64_t>(w.row_bytes), static_cast<std::uint64_t>(w.n),
                   static_cast<std::uint64_t>(w.row_bytes), Smem::kRowP, kTileN,
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
  p.magic = 0x43004300u;
  auto kernel = nbits_gemm_tcgen05_kernel<BT, BITS>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal) !=
      cudaSuccess) {
    return nullptr;
  }
  dim3 grid(static_cast<unsigned>((w.n + kTileN - 1) / kTileN),
            static_cast<unsigned>((m + BT - 1) / BT), 1);
  if (!LaunchBehindPrePass(kernel, grid, Smem::kTotal, stream, map_a, map_p, p)) {
    return nullptr;
  }
  CountLaunch();
  return BT == 256 ? "nbits_gemm_tcgen05_kernel<256>"
                   : (BT == 128 ? "nbits_gemm_tcgen05_kernel<128>" : "nbits_gemm_tcgen05_kernel<64>");
}

template <int BT>
const char *LaunchTile(const WeightView &w, std::int64_t m, const std::uint16_t *a_bf16, OutputView out,
                       int *status_word, cudaStream_t stream) {
  return w.bits == 8 ? LaunchTileBits<BT, 8>(w, m, a_bf16, out, status_word, stream)
                     : LaunchTileBits<BT, 4>(w, m, a_bf16, out, status_word, stream);
}

// Shape of a product on the pair kernel: token-tile width (a multiple of 16, at most 256) and the
// number of parts K is shared between; parts == 0 sends the product to the 128-row kernel instead.
// Chosen by a cost model in microseconds under load, fitted to measurements (N = 4096 ... 16032,
// K = 4096 and 14336, M = 17 ... 8192): a k step of a pair costs 0.30 + 0.0016 per token of the
// tile but at least 0.5 (the dequantization of 2 x 256 rows), a tile 4 for set-up plus 0.028 per
// token for its epilogue; the partial products of a shared K cross L2 once more on their way into Y
// (4 us + bytes at 4 TB/s); a k step of a tile of the 128-row kernel costs 0.375 and its tile 3.
struct PairPlan {
  int tokens;
  int parts;
};

PairPlan PairPlanFor(const WeightView &w, std::int64_t m, int sms, bool force_pair) {
  const std::int64_t pair_rows = (w.n + 2 * kPairRows - 1) / (2 * kPairRows);
  const std::int64_t slots = sms / 2 > 0 ? sms / 2 : 1;
  const std::int64_t k_steps = w.k / kTileK;
  PairPlan best{kPairTokens, 1};
  double best_cost = -1.0;
  for (int parts = 1; parts <= 8; parts *= 2) {
    if (parts > 1 && k_steps / parts < 8) {
      break;
    }
    const double steps = static_cast<double>((k_steps + parts - 1) / parts);
    for (int tokens = kPairTokens; tokens >= 64; tokens -= 16) {
      const std::int64_t tiles = pair_rows * ((m + tokens - 1) / tokens) * parts;
      const double rounds = static_cast<double>((tiles + slots - 1) / slots);
      const double step_cost = 0.30 + 0.0016 * tokens > 0.5 ? 0.30 + 0.0016 * tokens : 0.5;
      double cost = rounds * (4.0 + 0.028 * tokens + steps * step_cost);
      if (parts > 1) {
        cost += 4.0 + static_cast<double>(parts + 1) * static_cast<double>(m) * static_cast<double>(w.n) * 4.0 / 4.0e6;
      }
      if (best_cost < 0.0 || cost < best_cost) {
        best_cost = cost;
        best = PairPlan{tokens, parts};
      }
    }
  }
  if (!force_pair) {
    const std::int64_t tiles = ((w.n + kTileN - 1) / kTileN) * ((m + 127) / 128);
    const double rounds = static_cast<double>((tiles + sms - 1) / sms);
    if (rounds * (3.0 + 0.375 * static_cast<double>(k_steps)) < best_cost) {
      best.parts = 0;
    }
  }
  return best;
}

// Whether a product is considered for the pair kernel at all.
bool PairShape(const WeightView &w, std::int64_t m, bool force_pair) {
  return (w.bits == 4 || w.bits == 8) && (force_pair || m > 16);
}

template <int BITS>
const char *LaunchPairBits(const WeightView &w, std::int64_t m, const std::uint16_t *a_bf16, OutputView out,
                       int *status_word, cudaStream_t stream, int sms, float *partial, const PairPlan &plan) {
  const int tokens = plan.tokens;
  CUtensorMap map_a, map_p;
  if (!EncodeMap2D(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_bf16, static_cast<std::uint64_t>(w.k),
                   static_cast<std::uint64_t>(m), static_cast<std::uint64_t>(w.k) * 2, kTileK, tokens / 2,
                   CU_TENSOR_MAP_SWIZZLE_128B)) {
    return nullptr;
  }
  if (!EncodeMap2D(&map_p, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w.b, static_cast<std::uint64_t>(w.row_bytes),
                   static_cast<std::uint64_t>(w.n), static_cast<std::uint64_t>(w.row_bytes), PairSmem<BITS>::kRowP,
                   kPairRows, CU_TENSOR_MAP_SWIZZLE_NONE)) {
    return nullptr;
  }
  PairParams pp{};
  pp.g.w = w;
  pp.g.out = out;
  pp.g.m_total = static_cast<int>(m);
  pp.g.k_steps = static_cast<int>(w.k / kTileK);
  pp.g.status = status_word;
  pp.g.block_shift = Log2Of(w.block_size);
  pp.g.magic = 0x43004300u;
  pp.g.partial = plan.parts > 1 ? partial : nullptr;
  pp.tokens = tokens;
  pp.idesc = ptx::UmmaIdescBf16(256, tokens);
  auto kernel = nbits_gemm_tcgen05_pair_kernel<BITS>;
  constexpr int kPairSmem = PairSmem<BITS>::kTotal;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem) != cudaSuccess) {
    return nullptr;
  }
  const std::int64_t pair_rows = (w.n + 2 * kPairRows - 1) / (2 * kPairRows);
  dim3 grid(static_cast<unsigned>(2 * pair_rows), static_cast<unsigned>((m + tokens - 1) / tokens),
            static_cast<unsigned>(plan.parts));
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = dim3(kPairThreads, 1, 1);
  config.dynamicSmemBytes = kPairSmem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  if (cudaLaunchKernelEx(&config, kernel, map_a, map_p, pp) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  CountLaunch();
  if (plan.parts > 1) {
    const std::int64_t total = m * w.n;
    std::int64_t blocks = (total + 255) / 256;
    blocks = blocks > static_cast<std::int64_t>(sms) * 8 ? static_cast<std::int64_t>(sms) * 8 : blocks;
    if (!LaunchDependent(nbits_split_k_sum_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream,
                         static_cast<const float *>(partial), plan.parts, m, w.n, w.bias, out)) {
      return nullptr;
    }
    CountLaunch();
    return "nbits_gemm_tcgen05_pair_kernel(split-k)";
  }
  return "nbits_gemm_tcgen05_pair_kernel";
}

const char *LaunchPair(const WeightView &w, std::int64_t m, const std::uint16_t *a_bf16, OutputView out,
                       int *status_word, cudaStream_t stream, int sms, float *partial, const PairPlan &plan) {
  return w.bits == 8 ? LaunchPairBits<8>(w, m, a_bf16, out, status_word, stream, sms, partial, plan)
                     : LaunchPairBits<4>(w, m, a_bf16, out, status_word, stream, sms, partial, plan);
}

std::size_t AlignScratch(std::size_t v) { return (v + 255) & ~std::size_t{255}; }

} // namespace

// bf16 activations of one call, then (K shared between pairs only) the partial products [parts][m][n].
std::size_t GemmTcgen05ScratchBytes(const WeightView &w, std::int64_t m, int sm_count) {
  std::size_t bytes = AlignScratch(static_cast<std::size_t>(m) * static_cast<std::size_t>(w.k) * 2);
  if (PairShape(w, m, true)) {
    // the widest split either choice of kernel can take (the forced pair path may split where AUTO does not)
    const PairPlan forced = PairPlanFor(w, m, sm_count > 0 ? sm_count : 148, true);
    if (forced.parts > 1) {
      bytes += static_cast<std::size_t>(forced.parts) * static_cast<std::size_t>(m) * static_cast<std::size_t>(w.n) * sizeof(float);
    }
  }
  return bytes;
}

bool GemmTcgen05Supports(const WeightView &w, std::int64_t m) {
  return m >= 1 && (w.bits == 4 || w.bits == 8) && w.block_size >= 32 && (w.k % kTileK) == 0 &&
         (reinterpret_cast<std::uintptr_t>(w.b) & 15u) == 0 && (w.row_bytes % 16) == 0 &&
         GetEncodeTiled() != nullptr;
}

const char *LaunchGemmTcgen05(const WeightView &w, const float *a, std::int64_t m,
                              std::uint16_t *a_bf16, OutputView out, int *status_word,
                              cudaStream_t stream, int sm_count, int tiles) {
  if (!GemmTcgen05Supports(w, m) || (reinterpret_cast<std::uintptr_t>(a) & 15u) != 0) {
    return nullptr;
  }
  const std::int64_t groups = m * (w.k / 8);
  int blocks = static_cast<int>((groups + 255) / 256);
  const int max_blocks = (sm_count > 0 ? sm_count : 148) * 8;
  if (blocks > max_blocks) {
    blocks = max_blocks;
  }
  const int sms = sm_count > 0 ? sm_count : 148;
  if (!LaunchDependent(nbits_a_to_bf16_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, a, m, w.k,
                       reinterpret_cast<__nv_bfloat16 *>(a_bf16), w.bits == 4 ? 1 : 0)) {
    return nullptr;
  }
  CountLaunch();
  const std::int64_t n_tiles = (w.n + kTileN - 1) / kTileN;
  const bool force_pair = tiles == kGemmTilePairs;
  if (tiles != kGemmTileRows128 && PairShape(w, m, force_pair)) {
    const PairPlan plan = PairPlanFor(w, m, sms, force_pair);
    if (plan.parts >= 1) {
      float *partial = reinterpret_cast<float *>(
          reinterpret_cast<unsigned char *>(a_bf16) +
          AlignScratch(static_cast<std::size_t>(m) * static_cast<std::size_t>(w.k) * 2));
      const char *name = LaunchPair(w, m, a_bf16, out, status_word, stream, sms, partial, plan);
      if (name != nullptr) {
        return name;
      }
      cudaGetLastError();   // a cluster launch that the device refuses: the 128-row kernel takes the product
    }
  }
  // otherwise the widest token tile that still gives every SM a tile
  if (m > 128 && n_tiles * ((m + 255) / 256) >= sms) {
    return LaunchTile<256>(w, m, a_bf16, out, status_word, stream);
  }
  if (m > 64) {
    return LaunchTile<128>(w, m, a_bf16, out, status_word, stream);
  }
  return LaunchTile<64>(w, m, a_bf16, out, status_word, stream);
}

} // namespace mnb
