// How fast can ONE thread feed an SM with tensor copies?  148 (or 296) CTAs; 1, 2 or 4 producer threads per CTA issue
// ring-buffered cp.async.bulk.tensor loads behind mbarriers and only wait for them (no math).  Modes compare the box
// shapes / swizzles / access patterns the GEMM could use (weights in the [N/8][K/64][8][64] tile layout, activation limb
// planes [M][K]).  Loads only, every wait bounded.  What it showed on a B200: one thread's wait / expect_tx / copy round
// takes 0.3-0.4 us whatever the bytes, so small stages from a single producer cap a CTA far below what L2 delivers
// (8 KB stages: 3.9 TB/s over the GPU; the GEMM's old 16 KB stage of three copies: 4.6; a 32 KB stage of three copies: 8.5
// from one producer thread, 12.2 from two).  The GEMM's stage size and second producer thread follow from this.
//
// build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I tileinfer_b200/ops/csrc benchmarks/tma_issue_probe.cu -o benchmarks/tma_issue_probe -lcuda
// run:   benchmarks/tma_issue_probe        (prints one line per mode x producers x grid: time, GB/s)
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "tcgen05.cuh"

using namespace ti;

struct P {
  alignas(64) CUtensorMap map;
  alignas(64) CUtensorMap map2;
  int mode, iters, stage_bytes, stages, kb_count, tiles, nprod;
  unsigned* status;
};

// mode 0: weights-like 4D [n_tiles][KB][8][64] box {64,8,1,16}  (8 KB / load), CTA b walks kb for tile (b + j*grid)
// mode 1: 4D [n_tiles][KB/2][8][128] box {128,8,1,16} SW128 (16 KB / load)
// mode 2: limb-like 2D [64 rows][K] box {64, 64} SW64 (4 KB / load), every CTA reads the same rows
// mode 3: limb-like 2D [64 rows][K] box {128, 64} SW128 (8 KB / load)
// mode 4: plain 2D [rows][128] contiguous rows, box {128, 64} (8 KB contiguous)
__global__ void __launch_bounds__(128, 2) probe(const __grid_constant__ P p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t s0 = smem_u32(smem);
  const uint32_t bars = s0 + p.stages * p.stage_bytes;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) mbar_init(bars + 8 * s, 1);
    fence_mbar_init();
  }
  __syncthreads();
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) != 0 || w >= p.nprod) return;
  const int total = p.iters;
  int issued = w, done = w;                      // global load indices handled by this producer: w, w + nprod, ...
  while (done < total) {
    while (issued < total && issued - done < p.stages) {
      const int s = issued % p.stages;
      const int kb = issued % p.kb_count;
      int tile = blockIdx.x + (issued / p.kb_count) * gridDim.x;
      tile %= p.tiles;
      const uint32_t dst = s0 + s * p.stage_bytes, bar = bars + 8 * s;
      mbar_expect_tx(bar, p.stage_bytes);
      if (p.mode == 0 || p.mode == 1) {
        tma_load_4d(dst, &p.map, 0, 0, kb, tile * 16, bar);
      } else if (p.mode == 2) {
        tma_load_2d(dst, &p.map, kb * 64, 0, bar);
      } else if (p.mode == 3) {
        tma_load_2d(dst, &p.map, kb * 128, 0, bar);
      } else if (p.mode == 4) {
        tma_load_2d(dst, &p.map, 0, (tile * p.kb_count + kb) * 64, bar);
      } else if (p.mode == 5) {                      // the GEMM's stage at 64 tokens: 8 KB weights + 2 x 4 KB limbs
        tma_load_4d(dst, &p.map, 0, 0, kb, tile * 16, bar);
        tma_load_2d(dst + 8192, &p.map2, kb * 64, 0, bar);
        tma_load_2d(dst + 12288, &p.map2, kb * 64, 0, bar);
      } else if (p.mode == 6) {                      // the same with 128-byte rows: 16 KB weights + 2 x 8 KB limbs
        tma_load_4d(dst, &p.map, 0, 0, kb, tile * 16, bar);
        tma_load_2d(dst + 16384, &p.map2, kb * 128, 0, bar);
        tma_load_2d(dst + 24576, &p.map2, kb * 128, 0, bar);
      } else if (p.mode == 7) {                      // weights, 64-byte rows, two k slabs per copy (16 KB)
        tma_load_4d(dst, &p.map, 0, 0, kb * 2, tile * 16, bar);
      } else if (p.mode == 8) {                      // weights, 64-byte rows, four k slabs per copy (32 KB)
        tma_load_4d(dst, &p.map, 0, 0, kb * 4, tile * 16, bar);
      } else {                                       // mode 9: weights as in 7 + limbs with 128-byte rows (32 KB stage)
        tma_load_4d(dst, &p.map, 0, 0, kb * 2, tile * 16, bar);
        tma_load_2d(dst + 16384, &p.map2, kb * 128, 0, bar);
        tma_load_2d(dst + 24576, &p.map2, kb * 128, 0, bar);
      }
      issued += p.nprod;
    }
    const int s = done % p.stages;
    if (!mbar_wait(bars + 8 * s, (done / p.stages) & 1, 2000000000ull, p.status)) return;
    done += p.nprod;
  }
}

static int enc(CUtensorMap* m, void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
               CUtensorMapSwizzle sw) {
  cuuint32_t elem[4] = {1, 1, 1, 1};
  EncodeTiledFn e = encode_tiled_fn();
  CUresult r = e(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, base, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (int)r;
}

int main() {
  const int KB = 80, TILES = 592;                    // 592 tiles of 128 weight rows x 5120 B = 388 MB (> L2)
  const int n_tiles = TILES * 16;                    // row tiles of 8 rows
  const size_t wbytes = (size_t)n_tiles * KB * 512;  // 84.5 MB
  uint8_t* w;
  cudaMalloc(&w, wbytes * 2);                        // 2 copies, alternated
  cudaMemset(w, 1, wbytes * 2);
  uint8_t* x;
  const int K = KB * 64;
  cudaMalloc(&x, 64 * K);
  cudaMemset(x, 1, 64 * K);
  unsigned* status;
  cudaMalloc(&status, 4);
  cudaMemset(status, 0, 4);
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  for (int mode = 0; mode < 10; ++mode) {
   for (int nprod : {1, 2, 4}) {
    for (int grid : {148, 296}) {
      if (grid == 296 && nprod > 1) continue;
      P p = {};
      p.mode = mode;
      p.nprod = nprod;
      p.status = status;
      p.tiles = TILES;
      int loads_per_cta;
      std::vector<CUtensorMap> maps(2);
      for (int c = 0; c < 2; ++c) {
        uint8_t* base = w + c * wbytes;
        int r = 0;
        if (mode == 0 || mode == 5) {
          const cuuint64_t dims[4] = {64, 8, (cuuint64_t)KB, (cuuint64_t)n_tiles};
          const cuuint64_t strides[3] = {64, 512, (cuuint64_t)KB * 512};
          const cuuint32_t box[4] = {64, 8, 1, 16};
          r = enc(&maps[c], base, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
          p.stage_bytes = 8192; p.kb_count = KB;
        } else if (mode == 1 || mode == 6) {
          const cuuint64_t dims[4] = {128, 8, (cuuint64_t)KB / 2, (cuuint64_t)n_tiles};
          const cuuint64_t strides[3] = {128, 1024, (cuuint64_t)KB * 512};
          const cuuint32_t box[4] = {128, 8, 1, 16};
          r = enc(&maps[c], base, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
          p.stage_bytes = 16384; p.kb_count = KB / 2;
        } else if (mode == 7 || mode == 8 || mode == 9) {
          const cuuint32_t kk = mode == 8 ? 4 : 2;
          const cuuint64_t dims[4] = {64, 8, (cuuint64_t)KB, (cuuint64_t)n_tiles};
          const cuuint64_t strides[3] = {64, 512, (cuuint64_t)KB * 512};
          const cuuint32_t box[4] = {64, 8, kk, 16};
          r = enc(&maps[c], base, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
          p.stage_bytes = 8192 * kk; p.kb_count = KB / kk;
        } else if (mode == 2) {
          const cuuint64_t dims[2] = {(cuuint64_t)K, 64};
          const cuuint64_t strides[1] = {(cuuint64_t)K};
          const cuuint32_t box[2] = {64, 64};
          r = enc(&maps[c], x, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
          p.stage_bytes = 4096; p.kb_count = KB;
        } else if (mode == 3) {
          const cuuint64_t dims[2] = {(cuuint64_t)K, 64};
          const cuuint64_t strides[1] = {(cuuint64_t)K};
          const cuuint32_t box[2] = {128, 64};
          r = enc(&maps[c], x, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
          p.stage_bytes = 8192; p.kb_count = KB / 2;
        } else {
          const cuuint64_t dims[2] = {128, (cuuint64_t)(wbytes / 128)};
          const cuuint64_t strides[1] = {128};
          const cuuint32_t box[2] = {128, 64};
          r = enc(&maps[c], base, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
          p.stage_bytes = 8192; p.kb_count = KB;
        }
        if (mode == 5) {
          const cuuint64_t dims[2] = {(cuuint64_t)K, 64};
          const cuuint64_t strides[1] = {(cuuint64_t)K};
          const cuuint32_t box[2] = {64, 64};
          r |= enc(&p.map2, x, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
          p.stage_bytes = 16384;
        } else if (mode == 6 || mode == 9) {
          const cuuint64_t dims[2] = {(cuuint64_t)K, 64};
          const cuuint64_t strides[1] = {(cuuint64_t)K};
          const cuuint32_t box[2] = {128, 64};
          r |= enc(&p.map2, x, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
          p.stage_bytes = 32768;
        }
        if (r) { printf("encode failed mode %d: %d\n", mode, r); return 1; }
      }
      p.stages = (grid > 148 ? 96 : 192) * 1024 / p.stage_bytes;
      if (p.stages > 24) p.stages = 24;
      p.stages -= p.stages % nprod;
      loads_per_cta = p.kb_count * (TILES / grid);                  // one pass over the weight set
      p.iters = loads_per_cta;
      const size_t smem = (size_t)p.stages * p.stage_bytes + 8 * p.stages + 1024;
      float best = 1e9f, sum = 0.f;
      const int reps = 12;
      for (int it = 0; it < reps + 3; ++it) {
        p.map = maps[it % 2];
        cudaEventRecord(e0);
        probe<<<grid, 128, smem>>>(p);
        cudaEventRecord(e1);
        cudaEventSynchronize(e1);
        float ms;
        cudaEventElapsedTime(&ms, e0, e1);
        if (it >= 3) { best = ms < best ? ms : best; sum += ms; }
      }
      cudaError_t err = cudaGetLastError();
      unsigned st = 0;
      cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
      const double bytes = (double)grid * loads_per_cta * p.stage_bytes;
      printf("mode %d nprod %d grid %3d stage %5d B x %2d stages: %8.1f us avg %8.1f us best  %7.1f GB/s (avg)  err=%d status=%u\n", mode, nprod, grid,
             p.stage_bytes, p.stages, sum / reps * 1e3, best * 1e3, bytes / (sum / reps * 1e-3) / 1e9, (int)err, st);
    }
   }
  }
  return 0;
}
