// Stream-in ceilings of one B200 by load path: how fast can weights be brought from HBM into
// shared memory (or registers) with nothing else going on? Used to put the decode kernels'
// GB/s into context; it runs no MatMulNBits arithmetic.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 load_path_ceiling.cu -o load_path_ceiling -lcuda
//   ./load_path_ceiling
//
// Part 1, steady state over 1 GiB: (a) ld.global.cs.v4 from all threads, (b) 1-D bulk copies
// (cp.async.bulk) and (c) 2-D tiled TMA loads into a ring of shared-memory slots, by chunk size,
// ring depth, CTAs per SM and number of issuing threads per CTA.
// Part 2, short transfers: 32 MiB per launch (the size of one decode node), back-to-back
// launches over rotating parts of the buffer, including launch, ramp-up and tail.
// Every wait is bounded; a timed-out wait sets the status word that each line prints.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <vector>
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("ERR %s line %d\n", cudaGetErrorString(e_), __LINE__); exit(1);} } while (0)
__device__ __forceinline__ uint32_t sa(const void* p){ return (uint32_t)__cvta_generic_to_shared(p);} 
__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t c){ asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;"::"r"(sa(b)),"r"(c):"memory"); }
__device__ __forceinline__ void expect(uint64_t* b, uint32_t bytes){ asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"::"r"(sa(b)),"r"(bytes):"memory"); }
__device__ __forceinline__ bool trywait(uint64_t* b, uint32_t ph){ uint32_t d; asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0,1,0,p;\n}":"=r"(d):"r"(sa(b)),"r"(ph):"memory"); return d; }
__device__ __forceinline__ bool wait(uint64_t* b, uint32_t ph){ for (int i=0;i<(1<<20);++i){ if (trywait(b,ph)) return true; } return false; }
__device__ __forceinline__ void bulk(void* dst, const void* src, uint32_t bytes, uint64_t* b){ asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"::"r"(sa(dst)),"l"(src),"r"(bytes),"r"(sa(b)):"memory"); }
__device__ __forceinline__ void tma2d(void* dst, const void* map, int x, int y, uint64_t* b){ asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"::"r"(sa(dst)),"l"(map),"r"(x),"r"(y),"r"(sa(b)):"memory"); }

// mode 0: 1-D bulk copies of `chunk` bytes; mode 1: 2-D TMA box (chunk/16 bytes x 16 rows)
__global__ void __launch_bounds__(128) ring_kernel(const __grid_constant__ CUtensorMap map, const unsigned char* base, long long total_chunks, int chunk, int slots, int mode, int row_chunks, int issuers, int* status, unsigned* sink, int assign = 0) {
  extern __shared__ __align__(1024) unsigned char smem[];
  uint64_t* full = (uint64_t*)(smem + (size_t)slots * chunk);
  const int tid = threadIdx.x;
  if (tid == 0) { for (int s=0;s<slots;++s) mbar_init(&full[s],1); asm volatile("fence.mbarrier_init.release.cluster;":::"memory"); }
  __syncthreads();
  // chunks of this CTA: strided by grid
  // issuer threads: thread i*32 (i < issuers) handles slots s with s % issuers == i
  if ((tid & 31) == 0 && (tid >> 5) < issuers) {
    const int me = tid >> 5;
    long long mine = 0; // count of chunks this cta
    long long first = 0;
    if (assign == 0) { for (long long c = blockIdx.x; c < total_chunks; c += gridDim.x) ++mine; }
    else { first = blockIdx.x * total_chunks / gridDim.x; mine = (blockIdx.x + 1) * total_chunks / gridDim.x - first; }
    auto issue = [&](long long i) { // i-th chunk of this CTA
      const long long c = assign == 0 ? blockIdx.x + i * gridDim.x : first + i;
      const int s = (int)(i % slots);
      expect(&full[s], chunk);
      if (mode == 0) bulk(smem + (size_t)s*chunk, base + c * (long long)chunk, chunk, &full[s]);
      else { const long long tile = c / row_chunks; const int sl = (int)(c % row_chunks); tma2d(smem + (size_t)s*chunk, &map, sl * (chunk/16/4), (int)(tile*16), &full[s]); }
    };
    for (long long i = me; i < mine && i < slots; i += issuers) issue(i);
    unsigned acc = 0;
    for (long long i = me; i < mine; i += issuers) {
      const int s = (int)(i % slots);
      if (!wait(&full[s], (uint32_t)((i / slots) & 1))) { atomicExch(status, 1); break; }
      acc += *(volatile unsigned*)(smem + (size_t)s*chunk);
      if (i + slots < mine) issue(i + slots);
    }
    if (acc == 0x12345678u) *sink = acc;
  }
}

__global__ void __launch_bounds__(512) lsu_kernel(const uint4* base, long long n16, unsigned* sink) {
  unsigned acc = 0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 7 * stride < n16; i += 8 * stride) {
    uint4 v[8];
#pragma unroll
    for (int u=0;u<8;++u) v[u] = __ldcs(base + i + u*stride);
#pragma unroll
    for (int u=0;u<8;++u) acc += v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
  }
  if (acc == 0x12345678u) *sink = acc;
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int main() {
  const long long bytes = 1ll << 30; // 1 GiB
  unsigned char* buf; CK(cudaMalloc(&buf, bytes)); CK(cudaMemset(buf, 1, bytes));
  int* status; CK(cudaMalloc(&status, 4)); CK(cudaMemset(status, 0, 4));
  unsigned* sink; CK(cudaMalloc(&sink, 4));
  void* fp = nullptr; cudaDriverEntryPointQueryResult qr; CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fp, cudaEnableDefault, &qr));
  EncodeFn encode = (EncodeFn)fp;
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  auto timeit = [&](auto launch, const char* name) {
    launch(); CK(cudaDeviceSynchronize());
    float best = 1e9, sum = 0; const int reps = 5;
    for (int r=0;r<reps;++r){ cudaEventRecord(e0); launch(); cudaEventRecord(e1); CK(cudaDeviceSynchronize()); float ms; cudaEventElapsedTime(&ms,e0,e1); sum += ms; if (ms<best) best=ms; }
    int st; cudaMemcpy(&st,status,4,cudaMemcpyDeviceToHost);
    printf("%-52s mean %.1f GB/s best %.1f GB/s status %d\n", name, bytes/ (sum/reps*1e-3)/1e9, bytes/(best*1e-3)/1e9, st);
  };
  for (int ctas : {148*2, 148*4}) {
    char name[128]; snprintf(name, sizeof name, "lsu ldcs.v4 x8 unroll grid=%d x512", ctas);
    timeit([&]{ lsu_kernel<<<ctas,512>>>((const uint4*)buf, bytes/16, sink); }, name);
  }
  CK(cudaFuncSetAttribute(ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 225*1024));
  CUtensorMap dummy; memset(&dummy, 0, sizeof dummy);
  struct Cfg { int mode, chunk, slots, per_sm, row_bytes, issuers; };
  std::vector<Cfg> cfgs = {
    {0,16384,4,1,0,1},{0,16384,8,1,0,1},{0,16384,12,1,0,1},{0,16384,6,2,0,1},{0,8192,24,1,0,1},{0,32768,6,1,0,1},
    {0,16384,12,1,0,2},{0,16384,12,1,0,4},{0,4096,48,1,0,4},
    {1,16384,8,1,2048,1},{1,16384,12,1,2048,1},{1,16384,6,2,2048,1},{1,16384,12,1,1024,1},{1,16384,12,1,7168,1},{1,16384,12,1,2048,2},{1,16384,12,1,2048,4},{1,8192,24,1,2048,2},
  };
  for (auto c : cfgs) {
    CUtensorMap map = dummy; long long chunks = bytes / c.chunk; int row_chunks = 1;
    if (c.mode == 1) {
      const int box_w = c.chunk / 16; // bytes per row in box
      row_chunks = c.row_bytes / box_w;
      const cuuint64_t rows = bytes / c.row_bytes;
      cuuint64_t dims[2] = {(cuuint64_t)c.row_bytes/4, rows}; cuuint64_t strides[1] = {(cuuint64_t)c.row_bytes};
      cuuint32_t box[2] = {(cuuint32_t)box_w/4, 16}; cuuint32_t es[2] = {1,1};
      CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, buf, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); continue; }
    }
    char name[160]; snprintf(name, sizeof name, "%s chunk=%d slots=%d ctas/sm=%d row_bytes=%d issuers=%d", c.mode?"tma2d":"bulk1d", c.chunk, c.slots, c.per_sm, c.row_bytes, c.issuers);
    const size_t smem = (size_t)c.slots * c.chunk + 64 * 8;
    timeit([&]{ ring_kernel<<<148*c.per_sm,128,smem>>>(map, buf, chunks, c.chunk, c.slots, c.mode, row_chunks, c.issuers, status, sink); }, name);
  }

  // ---- short transfers: 32 MB per launch, rotating through the buffer, back-to-back launches ----
  {
    const long long part = 32ll << 20; const int parts = (int)(bytes / part);
    auto time_short = [&](auto launch, const char* name) {
      for (int i=0;i<parts;++i) launch(i); CK(cudaDeviceSynchronize());
      cudaEventRecord(e0); for (int r=0;r<4;++r) for (int i=0;i<parts;++i) launch(i); cudaEventRecord(e1); CK(cudaDeviceSynchronize());
      float ms; cudaEventElapsedTime(&ms,e0,e1); const double us = ms*1e3/(4*parts);
      int st; cudaMemcpy(&st,status,4,cudaMemcpyDeviceToHost);
      printf("%-60s %.2f us per 32 MB launch = %.1f GB/s status %d\n", name, us, part/(us*1e-6)/1e9, st);
    };
    time_short([&](int i){ lsu_kernel<<<148*2,512>>>((const uint4*)(buf + i*part), part/16, sink); }, "short lsu grid=296x512");
    for (int issuers : {1, 4}) for (int chunk : {16384, 8192}) {
      const int slots = 196608 / chunk;
      char name[128]; snprintf(name, sizeof name, "short bulk1d chunk=%d slots=%d issuers=%d", chunk, slots, issuers);
      const size_t smem = (size_t)slots * chunk + 64*8;
      time_short([&](int i){ ring_kernel<<<148,128,smem>>>(dummy, buf + i*part, part/chunk, chunk, slots, 0, 1, issuers, status, sink); }, name);
    }

    for (int assign : {0, 1}) for (int mode : {0, 1}) for (int chunk : {16384, 32768}) {
      if (mode == 1 && chunk != 16384) continue;
      const int slots = 196608 / chunk; const int issuers = 4;
      std::vector<CUtensorMap> maps(parts, dummy); int row_chunks = 1;
      if (mode == 1) {
        const int row_bytes = 2048; row_chunks = 2;
        for (int i = 0; i < parts; ++i) {
          cuuint64_t dims[2] = {(cuuint64_t)row_bytes/4, (cuuint64_t)(part/row_bytes)}; cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
          cuuint32_t box[2] = {256, 16}; cuuint32_t es[2] = {1,1};
          encode(&maps[i], CU_TENSOR_MAP_DATA_TYPE_INT32, 2, buf + i*part, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        }
      }
      char name[128]; snprintf(name, sizeof name, "short %s chunk=%d slots=%d issuers=4 assign=%s", mode?"tma2d(1KBx16 of 2KB rows)":"bulk1d", chunk, slots, assign?"contiguous":"strided");
      const size_t smem = (size_t)slots * chunk + 64*8;
      // 2-D mode addresses chunks relative to the whole buffer: offset by part index
      time_short([&](int i){ const long long c0 = (long long)i * (part/chunk); ring_kernel<<<148,128,smem>>>(maps[i], buf + i*part, part/chunk, chunk, slots, mode, row_chunks, issuers, status, sink, assign); (void)c0; }, name);
    }
    // empty kernel launch cost for reference
    time_short([&](int i){ lsu_kernel<<<148,512>>>((const uint4*)buf, 0, sink); }, "empty kernel (launch overhead only)");
  }
  return 0;
}
