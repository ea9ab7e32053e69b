// Load-path probe (diagnostic, not part of libqf_hotpath.so): how fast can the paged K/V tiles of ONE KV
// head be streamed on this GPU, with no math?  Pools are [pages,16,2,128] fp16, so a (page, head) tile is
// 16 rows of 256 B at a 512 B pitch.  Build and run:
//     nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 load_path_probe.cu -o load_path_probe
//     ./load_path_probe [pages=65536] [ctas_per_sm=2]
// Modes: 0 = 4-D tiled TMA box [1,16,1,128] per (page, head)   1 = TMA box [1,16,2,128] (whole page, both heads)
//        3 = cp.async.bulk, one 256-B row per copy              4 = per-thread 16-B cp.async + mbarrier arrive.noinc
//        2 = plain 16-B loads into registers
// Every wait is bounded.  No load uses a cluster-multicast qualifier.  Measured on B200: mode 0 3.73 TB/s,
// mode 1 6.5-6.8 TB/s, mode 3 1.6 TB/s, mode 4 4.6 (2 CTAs/SM) - 5.5 (3 CTAs/SM) TB/s, mode 2 6.7-6.9 TB/s.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <vector>
#include <algorithm>
#include <random>

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1);} } while (0)

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }" : "=r"(ok) : "r"(s32(bar)), "r"(parity) : "memory");
  return ok;
}
__device__ __forceinline__ bool wait_b(uint64_t* bar, uint32_t parity) {
  long long t0 = clock64();
  while (!try_wait(bar, parity)) { if (clock64() - t0 > 2000000000LL) return false; }
  return true;
}

constexpr int kStagesMax = 16;

// mode 0/1/3: each CTA streams tiles [first, last) of the tile list through a ring.
template <int MODE>
__global__ void __launch_bounds__(256) stream_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                              const unsigned char* kpool, const unsigned char* vpool,
                              const int* tiles /* page*2+head */, int tiles_per_cta, int stages, unsigned long long* sink, int* err) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ uint64_t full[kStagesMax], empty[kStagesMax];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int stage_bytes = MODE == 1 ? 16384 : 8192;  // K+V per tile
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(s32(&full[s])), "r"(MODE == 3 ? 1 : 1));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(s32(&empty[s])), "r"(8));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  const int* my = tiles + (size_t)blockIdx.x * tiles_per_cta;
  const int n = tiles_per_cta;
  unsigned long long acc = 0;
  int issued = 0;
  auto issue = [&](int i) {
    const int s = i % stages; const uint32_t par = ((i / stages) & 1) ^ 1;
    if (MODE == 3) {
      // warp 0: 32 lanes each copy one 256-B row (16 K rows + 16 V rows)
      if (lane == 0) { if (!wait_b(&empty[s], par)) *err = 1;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(s32(&full[s])), "r"(8192) : "memory"); }
      __syncwarp();
      const int t = my[i]; const int page = t >> 1, head = t & 1;
      const int r = lane & 15; const unsigned char* pool = lane < 16 ? kpool : vpool;
      const unsigned char* src = pool + ((size_t)page * 16 + r) * 512 + head * 256;
      unsigned char* dst = smem + s * stage_bytes + (lane < 16 ? 0 : 4096) + r * 256;
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   :: "r"(s32(dst)), "l"(src), "r"(256), "r"(s32(&full[s])) : "memory");
    } else if (lane == 0) {
      if (!wait_b(&empty[s], par)) *err = 1;
      const int t = my[i]; const int page = t >> 1, head = MODE == 1 ? 0 : (t & 1);
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(s32(&full[s])), "r"(stage_bytes) : "memory");
      unsigned char* dst = smem + s * stage_bytes;
      asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2,%3,%4,%5}], [%6];"
                   :: "r"(s32(dst)), "l"(&kmap), "r"(0), "r"(head), "r"(0), "r"(page), "r"(s32(&full[s])) : "memory");
      asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2,%3,%4,%5}], [%6];"
                   :: "r"(s32(dst + stage_bytes / 2)), "l"(&vmap), "r"(0), "r"(head), "r"(0), "r"(page), "r"(s32(&full[s])) : "memory");
    }
  };
  const int look = stages - 1;
  if (warp == 0) for (; issued < look && issued < n; ++issued) issue(issued);
  for (int i = 0; i < n; ++i) {
    if (warp == 0 && issued < n) { issue(issued); ++issued; }
    const int s = i % stages; const uint32_t par = (i / stages) & 1;
    if (!wait_b(&full[s], par)) { *err = 2; break; }
    acc += *reinterpret_cast<const unsigned int*>(smem + s * stage_bytes + tid * 16);
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(s32(&empty[s])) : "memory");
  }
  if (acc == 0x1234567ULL) sink[0] = acc;
}


// mode 4: every thread fills its own 16-B chunk of the K and V tile with cp.async (LDGSTS) and arrives on the
// stage's mbarrier when its copies land (cp.async.mbarrier.arrive.noinc); consumers wait on that barrier.
__global__ void __launch_bounds__(256) cpasync_kernel(const unsigned char* kpool, const unsigned char* vpool, const int* tiles,
                                                      int tiles_per_cta, int stages, unsigned long long* sink, int* err) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ uint64_t full[kStagesMax], empty[kStagesMax];
  const int tid = threadIdx.x, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(s32(&full[s])), "r"(256));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(s32(&empty[s])), "r"(8));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int* my = tiles + (size_t)blockIdx.x * tiles_per_cta;
  const int n = tiles_per_cta;
  const size_t thread_off = (size_t)(tid >> 4) * 512 + (tid & 15) * 16;
  unsigned long long acc = 0;
  int issued = 0;
  auto issue = [&](int i) {
    const int s = i % stages; const uint32_t par = ((i / stages) & 1) ^ 1;
    if (!wait_b(&empty[s], par)) *err = 1;
    const int t = my[i];
    const size_t off = (size_t)(t >> 1) * 8192 + (t & 1) * 256 + thread_off;
    const uint32_t dst = s32(smem + s * 8192 + tid * 16);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(kpool + off) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst + 4096), "l"(vpool + off) : "memory");
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" :: "r"(s32(&full[s])) : "memory");
  };
  const int look = stages - 1;
  for (; issued < look && issued < n; ++issued) issue(issued);
  for (int i = 0; i < n; ++i) {
    if (issued < n) { issue(issued); ++issued; }
    const int s = i % stages; const uint32_t par = (i / stages) & 1;
    if (!wait_b(&full[s], par)) { *err = 2; break; }
    acc += *reinterpret_cast<const unsigned int*>(smem + s * 8192 + tid * 16);
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(s32(&empty[s])) : "memory");
  }
  if (acc == 0x1234567ULL) sink[0] = acc;
}

// mode 2: plain loads, thread (t,c) of a 256-thread CTA loads its 16 B of K and V of each tile, 4 tiles in flight.
__global__ void __launch_bounds__(256) ldg_kernel(const unsigned char* kpool, const unsigned char* vpool, const int* tiles,
                                                  int tiles_per_cta, unsigned long long* sink) {
  const int tid = threadIdx.x; const int t = tid >> 4, c = tid & 15;
  const int* my = tiles + (size_t)blockIdx.x * tiles_per_cta;
  unsigned long long acc = 0;
  constexpr int U = 4;
  for (int i = 0; i + U <= tiles_per_cta; i += U) {
    uint4 k[U], v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int tl = my[i + u]; const size_t off = ((size_t)(tl >> 1) * 16 + t) * 512 + (tl & 1) * 256 + c * 16;
      k[u] = *reinterpret_cast<const uint4*>(kpool + off);
      v[u] = *reinterpret_cast<const uint4*>(vpool + off);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) acc += k[u].x + v[u].y;
  }
  if (acc == 0x1234567ULL) sink[0] = acc;
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int main(int argc, char** argv) {
  const int pages = argc > 1 ? atoi(argv[1]) : 65536;        // 8 KB per page per pool -> 512 MB per pool
  const int ctas_per_sm = argc > 2 ? atoi(argv[2]) : 2;
  const size_t pool_bytes = (size_t)pages * 8192;
  unsigned char *kpool, *vpool; CK(cudaMalloc(&kpool, pool_bytes)); CK(cudaMalloc(&vpool, pool_bytes));
  CK(cudaMemset(kpool, 1, pool_bytes)); CK(cudaMemset(vpool, 2, pool_bytes));
  const int sms = 148, grid = sms * ctas_per_sm;
  void* fn = nullptr; cudaDriverEntryPointQueryResult qr;
  CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr));
  EncodeFn encode = (EncodeFn)fn;
  auto make = [&](void* base, int box_heads, CUtensorMapL2promotion promo) {
    CUtensorMap m; cuuint64_t dims[4] = {128, 2, 16, (cuuint64_t)pages}; cuuint64_t strides[3] = {256, 512, 8192};
    cuuint32_t box[4] = {128, (cuuint32_t)box_heads, 16, 1}; cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult rc = encode(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) { printf("encode failed %d\n", (int)rc); exit(1); }
    return m;
  };
  unsigned long long* sink; CK(cudaMalloc(&sink, 8)); int* err; CK(cudaMalloc(&err, 4)); CK(cudaMemset(err, 0, 4));
  std::mt19937 rng(1);
  cudaEvent_t a, b; CK(cudaEventCreate(&a)); CK(cudaEventCreate(&b));
  for (int mode : {0, 1, 3, 4, 2}) {
    for (int order = 0; order < 2; ++order) {       // 0: random pages, 1: sequential pages
      for (int stages : {4, 8, 12}) {
        if (mode == 2 && stages != 4) continue;
        const int units = mode == 1 ? pages : pages * 2;  // tiles
        std::vector<int> tiles(units);
        if (mode == 1) for (int i = 0; i < units; ++i) tiles[i] = i * 2; else for (int i = 0; i < units; ++i) tiles[i] = i;
        if (order == 0) {
          if (mode == 1) std::shuffle(tiles.begin(), tiles.end(), rng);
          else { // shuffle pages, keep both heads of a page in different CTAs (head-major halves)
            std::vector<int> pg(pages); for (int i = 0; i < pages; ++i) pg[i] = i; std::shuffle(pg.begin(), pg.end(), rng);
            for (int i = 0; i < pages; ++i) { tiles[i] = pg[i] * 2; tiles[pages + i] = pg[(i * 7919) % pages] * 2 + 1; }
          }
        }
        const int per_cta = units / grid / 4 * 4;
        int* dtiles; CK(cudaMalloc(&dtiles, units * sizeof(int))); CK(cudaMemcpy(dtiles, tiles.data(), units * sizeof(int), cudaMemcpyHostToDevice));
        CUtensorMap km = make(kpool, mode == 1 ? 2 : 1, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        CUtensorMap vm = make(vpool, mode == 1 ? 2 : 1, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        const size_t smem = (size_t)stages * (mode == 1 ? 16384 : 8192);
        float best = 1e9;
        for (int rep = 0; rep < 4; ++rep) {
          CK(cudaEventRecord(a));
          if (mode == 0) { CK(cudaFuncSetAttribute(stream_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            stream_kernel<0><<<grid, 256, smem>>>(km, vm, kpool, vpool, dtiles, per_cta, stages, sink, err); }
          else if (mode == 1) { CK(cudaFuncSetAttribute(stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            stream_kernel<1><<<grid, 256, smem>>>(km, vm, kpool, vpool, dtiles, per_cta, stages, sink, err); }
          else if (mode == 3) { CK(cudaFuncSetAttribute(stream_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            stream_kernel<3><<<grid, 256, smem>>>(km, vm, kpool, vpool, dtiles, per_cta, stages, sink, err); }
          else if (mode == 4) { CK(cudaFuncSetAttribute(cpasync_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            cpasync_kernel<<<grid, 256, smem>>>(kpool, vpool, dtiles, per_cta, stages, sink, err); }
          else ldg_kernel<<<grid, 256>>>(kpool, vpool, dtiles, per_cta, sink);
          CK(cudaEventRecord(b)); CK(cudaEventSynchronize(b)); CK(cudaGetLastError());
          float ms; CK(cudaEventElapsedTime(&ms, a, b)); best = std::min(best, ms);
        }
        int herr; CK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
        const double bytes = (double)per_cta * grid * (mode == 1 ? 16384.0 : 8192.0);
        printf("mode %d %s stages %2d ctas/sm %d: %.3f ms  %.1f GB/s  err %d\n", mode, order ? "seq " : "rand", stages, ctas_per_sm,
               best, bytes / best / 1e6, herr);
        CK(cudaFree(dtiles));
      }
    }
  }
  return 0;
}
