// W8A16 GEMM for prefill (many activation rows): y[M, N] = x[M, K] * W[N, K]^T on the 5th-generation tensor
// cores (tcgen05.mma kind::i8, accumulators in tensor memory), fed by TMA.
//
// Replaces the reference's M > 1 path, which re-materialises a bf16 copy of the whole int8 weight on every
// call and hands it to cuBLAS (kernels/splitk_gemv.py:243-247).
//
// The int8 weights are multiplied as they are.  Each activation row is split exactly into two int8 limbs of
// a 16-bit fixed-point number with a per-row power-of-two exponent (x = (256*hi + lo) * 2^(e-14); hi signed,
// lo unsigned; `quant_rows_kernel`, which also fuses the RMSNorm(1+w) of the residual stream).  A CTA owns a
// 128 (weight rows) x 128 (tokens) output tile and keeps TWO int32 accumulators in TMEM (columns 0..127 for
// W*hi, 128..255 for W*lo); the epilogue combines them as (256*acc_hi + acc_lo) * 2^(e-14) * scale[row].
//
// Pipeline (192 threads): warp 0 = TMA producer (one elected lane): per 64-byte k slab one 4-D tensor copy
// of the weight tiles ([N/8][K/64][8][64] layout -> 128 rows x 64 B, 64-byte swizzle) and two 2-D copies of
// the limb planes; warp 1 = MMA issuer (one lane): four tcgen05.mma (2 k-steps x 2 limbs) per slab, then
// tcgen05.commit to release the stage; warps 2..5 = epilogue: tcgen05.ld of their 32 TMEM lanes, scale,
// fused epilogue (bf16 store / SwiGLU / residual add), coalesced stores.  8 stages of 24 KB.
// Every mbarrier wait is bounded; on expiry the status word is set, the roles drain and TMEM is freed.
#include <cuda.h>

#include "common.cuh"

namespace ti {

constexpr int kBM = 128;          // weight rows per CTA (TMEM lanes)
constexpr int kBN = 128;          // tokens per CTA (TMEM columns per accumulator)
constexpr int kBK = 64;           // bytes of k per stage (one 64-byte swizzle row)
constexpr int kGStages = 8;
constexpr int kStageA = kBM * kBK;                 // 8 KB
constexpr int kStageB = kBN * kBK;                 // 8 KB per limb plane
constexpr int kStageBytesG = kStageA + 2 * kStageB;
constexpr int kGemmThreads = 192;
constexpr unsigned long long kGemmWaitNs = 2000000000ull;

struct GemmParams {
  alignas(64) CUtensorMap map_w;   // uint8 [n_tiles][KB][8][64], box {64, 8, 1, 16}, 64B swizzle
  alignas(64) CUtensorMap map_xh;  // uint8 [M][K], box {64, 128}, 64B swizzle
  alignas(64) CUtensorMap map_xl;
  const float* xscale;             // [M] value of one fixed-point unit (2^(e-14))
  const __nv_bfloat16* wscale;     // [N_pad]
  const __nv_bfloat16* resid;      // ROWPAR: [M, N]
  void* out;                       // bf16 [M, ldo]  (SWIGLU: N/2 columns)
  unsigned* status;
  int M, N, K, ldo, epi;
};

// ---------------------------------------------------------------- PTX wrappers
TI_DEVICE bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred != 0;
}
TI_DEVICE void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
TI_DEVICE void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
TI_DEVICE void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_dst), "r"(cols) : "memory");
}
TI_DEVICE void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory"); }
TI_DEVICE void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}
TI_DEVICE void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
TI_DEVICE void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// D[tmem] (+)= A[smem desc] * B[smem desc], int8 operands, int32 accumulation, issued by one thread
TI_DEVICE void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on `bar` once all tcgen05.mma issued so far by this thread have completed
TI_DEVICE void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
TI_DEVICE void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
TI_DEVICE void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// K-major operand tile in shared memory, rows of 64 bytes, 64-byte swizzle, 8-row groups 512 bytes apart.
TI_DEVICE uint64_t smem_desc_sw64(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);            // start address, 16-byte units
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(512 >> 4) << 32;                     // stride byte offset: next 8-row group
  d |= (uint64_t)1 << 46;                              // descriptor version (Blackwell)
  d |= (uint64_t)4 << 61;                              // layout type: SWIZZLE_64B
  return d;
}
// kind::i8 instruction descriptor: D = s32, A = int8 (K-major), B = int8 / uint8 (K-major), M = 128, N = 128
TI_DEVICE constexpr uint32_t idesc_i8(bool b_signed) {
  return (2u << 4) | (1u << 7) | ((b_signed ? 1u : 0u) << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

enum { GEPI_STORE = 0, GEPI_SWIGLU = 1, GEPI_ROWPAR = 2 };

__global__ void __launch_bounds__(kGemmThreads, 1) gemm_w8a16_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // 1024-byte aligned stage buffers (the swizzle pattern repeats every 512 bytes)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t stage0 = smem_u32(smem);
  const uint32_t bars = stage0 + kGStages * kStageBytesG;       // full[8], empty[8], acc_full, tmem slot
  const uint32_t full0 = bars, empty0 = bars + 8 * kGStages, acc_bar = bars + 16 * kGStages, tmem_slot = acc_bar + 8;
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem + kGStages * kStageBytesG + 16 * kGStages + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_n = blockIdx.x, tile_m = blockIdx.y;
  const int KB = p.K / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(acc_bar, 1);
    fence_mbar_init();
  }
  if (warp == 1) {                       // one warp allocates 256 TMEM columns (two 128-column accumulators)
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      bool ok = true;
      for (int kb = 0; kb < KB && ok; ++kb) {
        const int s = kb % kGStages;
        const uint32_t par = ((kb / kGStages) & 1) ^ 1;           // a fresh barrier passes a wait on parity 1
        ok = mbar_wait(empty0 + 8 * s, par, kGemmWaitNs, p.status);
        if (!ok) break;
        const uint32_t dst = stage0 + s * kStageBytesG;
        mbar_expect_tx(full0 + 8 * s, kStageBytesG);
        tma_load_4d(dst, &p.map_w, 0, 0, kb, tile_n * (kBM / 8), full0 + 8 * s);
        tma_load_2d(dst + kStageA, &p.map_xh, kb * kBK, tile_m * kBN, full0 + 8 * s);
        tma_load_2d(dst + kStageA + kStageB, &p.map_xl, kb * kBK, tile_m * kBN, full0 + 8 * s);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      bool ok = true;
      for (int kb = 0; kb < KB && ok; ++kb) {
        const int s = kb % kGStages;
        ok = mbar_wait(full0 + 8 * s, (kb / kGStages) & 1, kGemmWaitNs, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a = stage0 + s * kStageBytesG, bh = a + kStageA, bl = bh + kStageB;
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {                          // two 32-byte k steps inside the 64-byte slab
          const uint64_t da = smem_desc_sw64(a + ks * 32);
          const uint32_t acc = (kb > 0 || ks > 0) ? 1u : 0u;
          umma_i8(tmem_base, da, smem_desc_sw64(bh + ks * 32), idesc_i8(true), acc);
          umma_i8(tmem_base + kBN, da, smem_desc_sw64(bl + ks * 32), idesc_i8(false), acc);
        }
        umma_commit(empty0 + 8 * s);                              // stage may be refilled once these MMAs are done
      }
      umma_commit(acc_bar);                                       // accumulators complete (or the loop gave up)
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 -> TMEM lane quarters)
    const int quarter = warp & 3;
    const bool ok = mbar_wait(acc_bar, 0, 2 * kGemmWaitNs, p.status);
    tc_fence_after();
    const int n = tile_n * kBM + quarter * 32 + lane;             // weight row == output feature of this lane
    const float ws = (ok && n < p.N) ? __bfloat162float(p.wscale[n]) : 0.f;
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    for (int c0 = 0; c0 < kBN; c0 += 32) {
      uint32_t hi[32], lo[32];
      tmem_ld32(taddr + c0, hi);
      tmem_ld32(taddr + kBN + c0, lo);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int m = tile_m * kBN + c0 + j;                      // token (uniform over the warp)
        if (m >= p.M) break;
        const float v = ((float)(int)hi[j] * 256.f + (float)(int)lo[j]) * p.xscale[m] * ws;
        if (p.epi == GEPI_SWIGLU) {
          // rows come interleaved (gate, up): lanes 2i / 2i+1
          const float other = __shfl_xor_sync(0xffffffffu, v, 1);
          if ((lane & 1) == 0 && n < p.N) {
            const float gate = round_bf16(v), up = round_bf16(other);
            static_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + (n >> 1)] = __float2bfloat16_rn(silu_f(gate) * up);
          }
        } else if (n < p.N) {
          float r = v;
          if (p.epi == GEPI_ROWPAR) r += __bfloat162float(p.resid[(size_t)m * p.N + n]);
          static_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + n] = __float2bfloat16_rn(r);
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// ---------------------------------------------------------------- activation limbs
// One block per row: optional RMSNorm(1+w), rounding to bf16, row maximum, quantisation to two int8 planes.
__global__ void __launch_bounds__(256) quant_rows_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                                         const __nv_bfloat16* __restrict__ norm_w, float eps, int K,
                                                         int8_t* __restrict__ xh, uint8_t* __restrict__ xl,
                                                         float* __restrict__ xscale) {
  __shared__ float red[8], bcast[2];
  const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const __nv_bfloat16* row = x + (size_t)m * ldx;
  float rr = 1.f;
  if (norm_w != nullptr) {
    float ss = 0.f;
    for (int k = tid; k < K; k += 256) {
      const float v = __bfloat162float(row[k]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
      for (int w = 0; w < 8; ++w) t += red[w];
      bcast[0] = rsqrtf(t / (float)K + eps);
    }
    __syncthreads();
    rr = bcast[0];
  }
  float mx = 0.f;
  for (int k = tid; k < K; k += 256) {
    float v = __bfloat162float(row[k]);
    if (norm_w != nullptr) v = round_bf16(v * rr * (1.f + __bfloat162float(norm_w[k])));
    mx = fmaxf(mx, fabsf(v));
  }
  mx = warp_max(mx);
  __syncthreads();
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (tid == 0) {
    float a = 0.f;
    for (int w = 0; w < 8; ++w) a = fmaxf(a, red[w]);
    int e = (int)((__float_as_uint(a) >> 23) & 0xffu) - 127;
    e = max(e, -100);
    if (!(a < 3.0e38f)) e = 127;
    bcast[1] = exp2f((float)(14 - e));
    xscale[m] = exp2f((float)(e - 14));
  }
  __syncthreads();
  const float qs = bcast[1];
  for (int k = tid; k < K; k += 256) {
    float v = __bfloat162float(row[k]);
    if (norm_w != nullptr) v = round_bf16(v * rr * (1.f + __bfloat162float(norm_w[k])));
    const int q = max(-32768, min(32767, __float2int_rn(v * qs)));
    xh[(size_t)m * K + k] = (int8_t)(q >> 8);
    xl[(size_t)m * K + k] = (uint8_t)(q & 0xff);
  }
}

// The driver entry point is resolved at run time, so the library also loads on machines without a driver.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

static int encode_map(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                      const cuuint32_t* box) {
  cuuint32_t elem[4] = {1, 1, 1, 1};
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return 999;
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(base), dims,
                                            strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

}  // namespace ti

extern "C" {

// xh/xl/xscale <- limbs of x (optionally RMS-normalised with (1+norm_w)); one launch, M blocks.
int ti_quant_rows(const void* x, int ldx, const void* norm_w, float eps, int M, int K, void* xh, void* xl, void* xscale,
                  void* stream) {
  if (M <= 0) return 0;
  ti::quant_rows_kernel<<<M, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)norm_w,
                                                             eps, K, (int8_t*)xh, (uint8_t*)xl, (float*)xscale);
  return (int)cudaGetLastError();
}

// y = x W^T for tiled int8 weights `w` ([n_tiles][K/64][8][64]) and the limb planes of x.
int ti_gemm_w8a16(const void* w, const void* wscale, int n_tiles, int N, int K, const void* xh, const void* xl,
                  const void* xscale, int M, const void* resid, void* out, int ldo, int epi, void* status, void* stream) {
  if (M <= 0) return 0;
  if (K % 64 || N < 1 || epi < 0 || epi > 2) return -2;
  ti::GemmParams p = {};
  const int KB = K / 64;
  {
    const cuuint64_t dims[4] = {64, 8, (cuuint64_t)KB, (cuuint64_t)n_tiles};
    const cuuint64_t strides[3] = {64, 512, (cuuint64_t)KB * 512};
    const cuuint32_t box[4] = {64, 8, 1, 16};
    const int rc = ti::encode_map(&p.map_w, w, 4, dims, strides, box);
    if (rc) return rc;
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K};
    const cuuint32_t box[2] = {64, 128};
    int rc = ti::encode_map(&p.map_xh, xh, 2, dims, strides, box);
    if (rc) return rc;
    rc = ti::encode_map(&p.map_xl, xl, 2, dims, strides, box);
    if (rc) return rc;
  }
  p.xscale = (const float*)xscale;
  p.wscale = (const __nv_bfloat16*)wscale;
  p.resid = (const __nv_bfloat16*)resid;
  p.out = out;
  p.status = (unsigned*)status;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldo = ldo;
  p.epi = epi;
  const size_t smem = (size_t)ti::kGStages * ti::kStageBytesG + 16 * ti::kGStages + 64 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(ti::gemm_w8a16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = true;
  }
  dim3 grid((n_tiles * 8 + ti::kBM - 1) / ti::kBM, (M + ti::kBN - 1) / ti::kBN);
  ti::gemm_w8a16_kernel<<<grid, ti::kGemmThreads, smem, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}

}  // extern "C"
