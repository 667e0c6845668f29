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
// Pipeline (224 threads): warps 0 and 6 = TMA producers (one elected lane each, alternate stages): per stage of
// 128 bytes of k one 4-D tensor copy of the weight tiles ([N/8][K/64][8][64] layout -> per row tile the 8 x 64-byte
// rows of two k slabs, 64-byte swizzle) and two 2-D copies of the limb planes (rows of 128 bytes, 128-byte swizzle);
// warp 1 = MMA issuer (one lane): eight tcgen05.mma (4 k-steps x 2 limbs) per stage and 128-row half, then
// tcgen05.commit to release the stage; warps 2..5 = epilogue: tcgen05.ld of their 32 TMEM lanes, scale,
// fused epilogue (bf16 store / SwiGLU / residual add), coalesced stores.
// Stage size and the second producer come from measurement: one thread's wait / expect_tx / copy sequence takes
// ~0.4 us whatever the bytes, so 16 KB stages from one thread cap a CTA at ~40 GB/s (5.9 TB/s over the GPU, operands
// included), below what the tensor pipe (many tokens) or HBM (few tokens) would take; 32-64 KB stages from two
// threads lift the cap to ~12 TB/s.
// The token tile is a template parameter (32, 64 or 128 tokens): a decode batch of 17..64 rows then moves 4-8 KB of
// limbs per 8 KB of weights instead of 16 KB, and the ring holds 12-16 stages, so the kernel streams weights at
// HBM speed.  Products with few weight-row tiles (N = 5120: 40 tiles for 148 SMs) are split along k over
// gridDim.z; the scaled fp32 partials meet in a workspace and the last CTA of a tile to arrive adds them in split
// order (deterministic) and runs the epilogue.
// Every mbarrier wait is bounded; on expiry the status word is set, the roles drain and TMEM is freed.
#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

#include "tcgen05.cuh"

namespace ti {

constexpr int kBM = 128;          // weight rows per CTA (TMEM lanes)
constexpr int kBK = 64;           // bytes of k per weight slab (one 64-byte swizzle row)
constexpr int kKS = 2;            // weight slabs per stage: one stage = 128 bytes of k
constexpr int kStageA = kBM * kBK * kKS;           // 16 KB of weights per stage and 128-row half
constexpr int kGemmThreads = 224;      // warp 0 and warp 6: TMA producers; warp 1: MMA issuer; warps 2..5: epilogue
constexpr int kGemmProducerB = 6;
#ifndef TI_GEMM_RING_KB
#define TI_GEMM_RING_KB 192
#endif
// bytes of operand ring per CTA.  96 lets two CTAs share an SM (TMEM: 2 x 256 columns), so that the epilogue of
// one overlaps the main loop of the other.
constexpr int kGemmRingBytes = TI_GEMM_RING_KB * 1024;
// BN = tokens per CTA (TMEM columns per accumulator); BF16: bf16 weights and activations (one plane, one accumulator)
// BMH = weight-row halves per CTA: 1 -> a 128-row tile; 2 -> a 256-row tile as two 128-row MMAs that share ONE
// activation tile in shared memory (the bytes a CTA pulls through L2 per multiply-add drop by a third).
template <int BN, bool BF16, int BMH = 1> struct GemmGeom {
  static constexpr int kStageB = BN * kBK * kKS;                   // one limb plane / the bf16 activation tile (128-byte rows)
  static constexpr int kStageBytes = BMH * kStageA + (BF16 ? 1 : 2) * kStageB;
  static constexpr int kStages = kGemmRingBytes / kStageBytes < 24 ? kGemmRingBytes / kStageBytes : 24;
  static constexpr size_t kSmem = (size_t)kStages * kStageBytes + 16 * kStages + 64 + 1024;
};
constexpr unsigned long long kGemmWaitNs = 2000000000ull;

struct GemmParams {
  alignas(64) CUtensorMap map_w;   // uint8 [n_tiles][KB][8][64], box {64, 8, 2, 16 or 32}, 64B swizzle
  alignas(64) CUtensorMap map_xh;  // uint8 [M][K], box {128, BN}, 128B swizzle (bf16 mode: the activations, [M][2K] bytes)
  alignas(64) CUtensorMap map_xl;
  const float* xscale;             // [M] value of one fixed-point unit (2^(e-14))
  const __nv_bfloat16* wscale;     // [N_pad]
  const __nv_bfloat16* resid;      // ROWPAR: [M, N]
  void* out;                       // bf16 [M, ldo]  (SWIGLU: N/2 columns)
  unsigned* status;
  float* part;                     // split-k partials [S][M][N] fp32
  unsigned* tile_count;            // [tiles_n * tiles_m] arrival counters, zero between launches
  int M, N, K, ldo, epi;
  int kb_per_split;                // 128-byte k stages per gridDim.z slice
  int ablate;                      // timing experiments only (TI_GEMM_ABLATE): 1 no MMA, 2 no activation copies, 4 no weight copies, 8 no epilogue, 16 no main loop, 32 no split-k reduction, 64 no fence before the split-k count
};

// kind::i8 instruction descriptor: D = s32, A = int8 (K-major), B = int8 / uint8 (K-major), M = 128, N = BN
template <int BN> TI_DEVICE constexpr uint32_t idesc_i8(bool b_signed) {
  return (2u << 4) | (1u << 7) | ((b_signed ? 1u : 0u) << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

// kind::f16 instruction descriptor: D = f32, A = B = bf16 (K-major), M = 128, N = BN
template <int BN> TI_DEVICE constexpr uint32_t idesc_bf16() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

enum { GEPI_STORE = 0, GEPI_SWIGLU = 1, GEPI_ROWPAR = 2, GEPI_F32 = 3 };

// fused epilogue for four adjacent weight rows n..n+3 of one token (N is a multiple of 4 here): split-k reduction
TI_DEVICE void gemm_epilogue4(const GemmParams& p, int m, int n, float4 v, uint2 r) {
  if (p.epi == GEPI_SWIGLU) {
    const float g0 = round_bf16(v.x), u0 = round_bf16(v.y), g1 = round_bf16(v.z), u1 = round_bf16(v.w);
    *reinterpret_cast<uint32_t*>(static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldo + (n >> 1)) =
        pack_bf16(silu_f(g0) * u0, silu_f(g1) * u1);
    return;
  }
  if (p.epi == GEPI_F32) {
    *reinterpret_cast<float4*>(static_cast<float*>(p.out) + (size_t)m * p.ldo + n) = v;
    return;
  }
  if (p.epi == GEPI_ROWPAR) {                      // r: the residual row's four values, loaded by the caller
    v.x += bf16lo(r.x);
    v.y += bf16hi(r.x);
    v.z += bf16lo(r.y);
    v.w += bf16hi(r.y);
  }
  *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldo + n) =
      make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

// Eight adjacent weight rows n..n+7 (n a multiple of 8) of one token, straight from the accumulators: split-k
// partial (fp32), or the fused epilogue.  Rows past N and rows that cannot be stored as one vector go one by one.
TI_DEVICE void gemm_store8(const GemmParams& p, int m, int n, const float4 a, const float4 b, int S, int split) {
  const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  if (S > 1) {
    float* dst = p.part + ((size_t)split * p.M + m) * p.N + n;
    if (n + 8 <= p.N) {
      *reinterpret_cast<float4*>(dst) = a;
      *reinterpret_cast<float4*>(dst + 4) = b;
    } else {
      for (int i = 0; i < 8 && n + i < p.N; ++i) dst[i] = v[i];
    }
    return;
  }
  const bool full = n + 8 <= p.N;
  if (p.epi == GEPI_SWIGLU) {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldo + (n >> 1);
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = silu_f(round_bf16(v[2 * i])) * round_bf16(v[2 * i + 1]);
    if (full && (p.ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 7) == 0) {
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
    } else {
      for (int i = 0; i < 4 && n + 2 * i < p.N; ++i) dst[i] = __float2bfloat16_rn(o[i]);
    }
    return;
  }
  if (p.epi == GEPI_F32) {
    float* dst = static_cast<float*>(p.out) + (size_t)m * p.ldo + n;
    if (full && (p.ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) {
      *reinterpret_cast<float4*>(dst) = a;
      *reinterpret_cast<float4*>(dst + 4) = b;
    } else {
      for (int i = 0; i < 8 && n + i < p.N; ++i) dst[i] = v[i];
    }
    return;
  }
  float r[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) r[i] = v[i];
  const bool vec = full && (p.ldo & 7) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 &&
                   (p.epi != GEPI_ROWPAR || ((p.N & 7) == 0 && (reinterpret_cast<uintptr_t>(p.resid) & 15) == 0));
  if (p.epi == GEPI_ROWPAR) {
    const __nv_bfloat16* rs = p.resid + (size_t)m * p.N + n;
    if (vec) {
      const uint4 q = *reinterpret_cast<const uint4*>(rs);
      const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) { r[2 * i] += bf16lo(w4[i]); r[2 * i + 1] += bf16hi(w4[i]); }
    } else {
      for (int i = 0; i < 8 && n + i < p.N; ++i) r[i] += __bfloat162float(rs[i]);
    }
  }
  __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldo + n;
  if (vec) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16(r[0], r[1]), pack_bf16(r[2], r[3]), pack_bf16(r[4], r[5]), pack_bf16(r[6], r[7]));
  } else {
    for (int i = 0; i < 8 && n + i < p.N; ++i) dst[i] = __float2bfloat16_rn(r[i]);
  }
}

template <int BN, bool BF16, int BMH>
__global__ void __launch_bounds__(kGemmThreads, TI_GEMM_RING_KB <= 100 ? 2 : 1) gemm_w8a16_kernel(const __grid_constant__ GemmParams p) {
  using G = GemmGeom<BN, BF16, BMH>;
  constexpr int kAcc = BF16 ? 1 : 2;                               // accumulators (limbs) per row half
  constexpr int kStages = G::kStages, kStageBytes = G::kStageBytes, kStageB = G::kStageB;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // 1024-byte aligned stage buffers (the swizzle pattern repeats every 512 bytes)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t stage0 = smem_u32(smem);
  const uint32_t bars = stage0 + kStages * kStageBytes;         // full[], empty[], acc_full, tmem slot
  const uint32_t full0 = bars, empty0 = bars + 8 * kStages, acc_bar = bars + 16 * kStages, tmem_slot = acc_bar + 8;
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem + kStages * kStageBytes + 16 * kStages + 8);
  __shared__ int s_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // token tiles vary fastest: the CTAs that run at the same time share weight tiles (read from HBM once, then L2
  // hits) and the limb planes of all tokens stay in L2
  const int tile_m = blockIdx.x, tile_n = blockIdx.y, split = blockIdx.z, S = gridDim.z;
  const int KB = (p.K + kBK * kKS - 1) / (kBK * kKS);               // stages of 128 bytes of k (a last half stage reads zeros)
  const int kb0 = split * p.kb_per_split, kb1 = (p.ablate & 16) ? kb0 : min(KB, kb0 + p.kb_per_split);
  constexpr uint32_t kCols = BMH * kAcc * BN < 32 ? 32 : BMH * kAcc * BN;   // TMEM allocation: a power of two >= 32

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(acc_bar, 1);
    fence_mbar_init();
  }
  if (warp == 1) {                       // one warp allocates the TMEM columns of the two accumulators
    tmem_alloc(tmem_slot, kCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  pdl_trigger();
  if (warp == 0 || warp == kGemmProducerB) {
    // ------------------------------------------------------------ TMA producers
    // Two producer threads (in two warps) take the stages alternately: one thread's wait / expect / copy sequence
    // takes ~0.4 us per stage, which is less than the ring can absorb.  The weights of the first ring fill do not
    // depend on the preceding kernel: they are requested before the programmatic-dependency wait, the activations
    // (written by that kernel) after it.
    const int first = warp == 0 ? 0 : 1;
    const int n_it = kb1 - kb0, n_pre = min(kStages, n_it);
    const uint32_t stage_tx = ((p.ablate & 4) ? 0 : BMH * kStageA) + ((p.ablate & 2) ? 0 : (BF16 ? 1 : 2) * kStageB) + ((p.ablate & 6) == 6 ? 0 : 0);
    if (elect_one()) {
      for (int it = first; it < n_pre; it += 2) {
        mbar_expect_tx(full0 + 8 * it, stage_tx);
        if (!(p.ablate & 4)) tma_load_4d(stage0 + it * kStageBytes, &p.map_w, 0, 0, (kb0 + it) * kKS, tile_n * (BMH * kBM / 8), full0 + 8 * it);
      }
    }
    __syncwarp();
    pdl_wait();
    if (elect_one()) {
      for (int it = first; it < n_pre; it += 2) {
        const uint32_t dst = stage0 + it * kStageBytes;
        if (p.ablate & 2) continue;
        tma_load_2d(dst + BMH * kStageA, &p.map_xh, (kb0 + it) * kBK * kKS, tile_m * BN, full0 + 8 * it);
        if (!BF16) tma_load_2d(dst + BMH * kStageA + kStageB, &p.map_xl, (kb0 + it) * kBK * kKS, tile_m * BN, full0 + 8 * it);
      }
      int it = n_pre + ((n_pre & 1) == first ? 0 : 1);            // this producer's first stage after the pre-fill
      for (; it < n_it; it += 2) {
        const int s = it % kStages, kb = kb0 + it;
        const uint32_t par = ((it / kStages) & 1) ^ 1;            // a fresh barrier passes a wait on parity 1
        if (!mbar_wait(empty0 + 8 * s, par, kGemmWaitNs, p.status)) break;
        const uint32_t dst = stage0 + s * kStageBytes;
        mbar_expect_tx(full0 + 8 * s, stage_tx);
        if (!(p.ablate & 4)) tma_load_4d(dst, &p.map_w, 0, 0, kb * kKS, tile_n * (BMH * kBM / 8), full0 + 8 * s);   // box: 2 slabs x BMH * 16 row tiles
        if (p.ablate & 2) continue;
        tma_load_2d(dst + BMH * kStageA, &p.map_xh, kb * kBK * kKS, tile_m * BN, full0 + 8 * s);
        if (!BF16) tma_load_2d(dst + BMH * kStageA + kStageB, &p.map_xl, kb * kBK * kKS, tile_m * BN, full0 + 8 * s);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    pdl_wait();
    if (elect_one()) {
      bool ok = true;
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        const int it = kb - kb0, s = it % kStages;
        ok = mbar_wait(full0 + 8 * s, (it / kStages) & 1, kGemmWaitNs, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a = stage0 + s * kStageBytes, bh = a + BMH * kStageA, bl = bh + kStageB;
#pragma unroll
        for (int j = 0; j < 2 * kKS; ++j) {                       // four 32-byte k steps inside the 128 bytes of the stage
          if (p.ablate & 1) break;
          const uint32_t acc = (it > 0 || j > 0) ? 1u : 0u;
          // activations: rows of 128 bytes (128-byte swizzle); weights: per row tile the 8 x 64-byte rows of slab 0,
          // then those of slab 1 (64-byte swizzle, 8-row groups 1024 bytes apart)
          const uint64_t dbh = smem_desc_sw128(bh + j * 32), dbl = smem_desc_sw128(bl + j * 32);
#pragma unroll
          for (int h = 0; h < BMH; ++h) {                         // the row halves share the activation operand
            const uint64_t da = smem_desc_sw64_sbo(a + h * kStageA + (j >> 1) * 512 + (j & 1) * 32, 1024);
            const uint32_t d0 = tmem_base + (uint32_t)(h * kAcc * BN);
            if (BF16) {
              umma_bf16(d0, da, dbh, idesc_bf16<BN>(), acc);
            } else {
              umma_i8(d0, da, dbh, idesc_i8<BN>(true), acc);
              umma_i8(d0 + BN, da, dbl, idesc_i8<BN>(false), acc);
            }
          }
        }
        umma_commit(empty0 + 8 * s);                              // stage may be refilled once these MMAs are done
      }
      umma_commit(acc_bar);                                       // accumulators complete (or the loop gave up)
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 -> TMEM lane quarters)
    const int quarter = warp & 3;
    pdl_wait();
    const bool ok = mbar_wait(acc_bar, 0, 2 * kGemmWaitNs, p.status);
    tc_fence_after();
    // The operand ring is idle now (every copy has landed and every MMA has read its operands): each warp stages
    // a 32-token x 32-row block of results there (fp32, 36-float pitch: conflict-free both ways) and writes it out
    // with 8 rows = 16 bytes of bf16 per thread, 8 tokens per instruction, instead of 2 bytes per thread.
    float* stage_t = reinterpret_cast<float*>(smem) + (warp - 2) * (32 * 36);
#pragma unroll 1
    for (int h = 0; h < BMH; ++h) {
      const int n0 = tile_n * (BMH * kBM) + h * kBM + quarter * 32;           // first weight row of this warp's block
      const int n = n0 + lane;                                                 // weight row == output feature of this lane
      const float ws = (ok && n < p.N) ? (BF16 ? 1.f : __bfloat162float(p.wscale[n])) : 0.f;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(h * kAcc * BN);
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (p.ablate & 8) break;
        if (tile_m * BN + c0 >= p.M) break;
        uint32_t hi[32], lo[32];
        tmem_ld32(taddr + c0, hi);
        if (!BF16) tmem_ld32(taddr + BN + c0, lo);
        // the row scales of the 32 tokens of this chunk: one coalesced load, handed round by shuffles
        const int m_lane = tile_m * BN + c0 + lane;
        const float xs_lane = (!BF16 && m_lane < p.M) ? p.xscale[m_lane] : 0.f;
        tmem_ld_wait();
        __syncwarp();                                                          // the previous block has been written out
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float xs = __shfl_sync(0xffffffffu, xs_lane, j);
          stage_t[j * 36 + lane] = BF16 ? __uint_as_float(hi[j]) * ws
                                        : ((float)(int)hi[j] * 256.f + (float)(int)lo[j]) * xs * ws;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int t = (lane >> 2) + 8 * i, c = lane & 3;
          const int m = tile_m * BN + c0 + t;
          if (m < p.M && n0 + c * 8 < p.N) {
            const float4 a = *reinterpret_cast<const float4*>(stage_t + t * 36 + c * 8);
            const float4 b = *reinterpret_cast<const float4*>(stage_t + t * 36 + c * 8 + 4);
            gemm_store8(p, m, n0 + c * 8, a, b, S, split);
          }
        }
      }
    }
    tc_fence_before();
  }
  if (S > 1) {
    // ---- split-k: the last CTA of this output tile to arrive adds the partials in split order
    if (!(p.ablate & 64)) __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned prev = atomicAdd(p.tile_count + tile_n * gridDim.x + tile_m, 1u);
      s_last = prev + 1 == (unsigned)S;
      if (s_last) p.tile_count[tile_n * gridDim.x + tile_m] = 0;   // ready for the next launch
      __threadfence();
    }
    __syncthreads();
    if (s_last && warp >= 2 && warp < 6 && !(p.ablate & 32)) {
      // lane -> four adjacent output features, warp -> every fourth token.  The partial sums of four tokens and four
      // slices (and the residual rows) are requested together before the first is used: with the loads inside a
      // loop of run-time length each one waited for the one before it (12 memory round trips per four tokens; the
      // reduction of a 64-token tile took 27 us).  The slices are added in ascending order whatever the grouping.
      const int m_end = min(p.M, (tile_m + 1) * BN);
      for (int hh = 0; hh < BMH; ++hh) {
      const int n4 = tile_n * (BMH * kBM) + hh * kBM + lane * 4;
      if (n4 >= p.N) continue;
      for (int m0 = tile_m * BN + (warp - 2); m0 < m_end; m0 += 16) {
        float4 acc[4];
        uint2 rs[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          rs[u] = make_uint2(0u, 0u);
          const int m = m0 + 4 * u;
          if (m < m_end && p.epi == GEPI_ROWPAR) rs[u] = __ldcg(reinterpret_cast<const uint2*>(p.resid + (size_t)m * p.N + n4));
        }
        for (int z0 = 0; z0 < S; z0 += 4) {
          float4 v[4][4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int zz = 0; zz < 4; ++zz) {
              const int m = m0 + 4 * u, z = z0 + zz;
              v[u][zz] = (m < m_end && z < S) ? __ldcg(reinterpret_cast<const float4*>(p.part + ((size_t)z * p.M + m) * p.N + n4))
                                              : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int zz = 0; zz < 4; ++zz) {
              acc[u].x += v[u][zz].x;
              acc[u].y += v[u][zz].y;
              acc[u].z += v[u][zz].z;
              acc[u].w += v[u][zz].w;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int m = m0 + 4 * u;
          if (m < m_end) gemm_epilogue4(p, m, n4, acc[u], rs[u]);
        }
      }
      }
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kCols);
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

// The same for rows of up to 512 * 5 * 8 = 20480 elements in ONE pass: every thread keeps its (up to five) 16-byte
// chunks of the row in registers between the statistics and the quantisation, so the row is read once.  The block is
// as small as the row allows (K / 40 threads, rounded up to warps: 128 threads at K = 5120), so that many rows are in
// flight per SM: a row is a load -> reduce -> reduce -> store chain of a few microseconds, and 8192 rows of 512 threads
// each pass through an SM only four at a time.
__global__ void __launch_bounds__(512) quant_rows_fast_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                                              const __nv_bfloat16* __restrict__ norm_w, float eps, int K,
                                                              int8_t* __restrict__ xh, uint8_t* __restrict__ xl,
                                                              float* __restrict__ xscale) {
  __shared__ float red[16], red2[16];
  const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const __nv_bfloat16* row = x + (size_t)m * ldx;
  const int nchunk = K >> 3;
  const int nthr = blockDim.x, nwarp = nthr >> 5;
  pdl_trigger();
  pdl_wait();
  float v[5][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 5; ++j) {
    const int c = tid + j * nthr;
    uint4 q = make_uint4(0, 0, 0, 0);
    if (c < nchunk) q = *reinterpret_cast<const uint4*>(row + (size_t)c * 8);
    const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[j][2 * i] = bf16lo(w4[i]);
      v[j][2 * i + 1] = bf16hi(w4[i]);
      ss += v[j][2 * i] * v[j][2 * i] + v[j][2 * i + 1] * v[j][2 * i + 1];
    }
  }
  if (norm_w != nullptr) {
    uint4 nwv[5];
#pragma unroll
    for (int j = 0; j < 5; ++j) {
      const int c = tid + j * nthr;
      nwv[j] = c < nchunk ? *reinterpret_cast<const uint4*>(norm_w + (size_t)c * 8) : make_uint4(0, 0, 0, 0);
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 16; ++w) tot += w < nwarp ? red[w] : 0.f;
    const float rr = rsqrtf(tot / (float)K + eps);
#pragma unroll
    for (int j = 0; j < 5; ++j) {
      const uint32_t n4[4] = {nwv[j].x, nwv[j].y, nwv[j].z, nwv[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[j][2 * i] = round_bf16(v[j][2 * i] * rr * (1.f + bf16lo(n4[i])));
        v[j][2 * i + 1] = round_bf16(v[j][2 * i + 1] * rr * (1.f + bf16hi(n4[i])));
      }
    }
  }
  float mx = 0.f;
#pragma unroll
  for (int j = 0; j < 5; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(v[j][i]));
  mx = warp_max(mx);
  if (lane == 0) red2[warp] = mx;
  __syncthreads();
  float a = 0.f;
#pragma unroll
  for (int w = 0; w < 16; ++w) a = fmaxf(a, w < nwarp ? red2[w] : 0.f);
  int e = (int)((__float_as_uint(a) >> 23) & 0xffu) - 127;
  e = max(e, -100);
  if (!(a < 3.0e38f)) e = 127;
  const float qs = exp2f((float)(14 - e));
  if (tid == 0) xscale[m] = exp2f((float)(e - 14));
#pragma unroll
  for (int j = 0; j < 5; ++j) {
    const int c = tid + j * nthr;
    if (c >= nchunk) continue;
    uint32_t hw[2] = {0, 0}, lw[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q = max(-32768, min(32767, __float2int_rn(v[j][i] * qs)));
      hw[i >> 2] |= (uint32_t)((q >> 8) & 0xff) << (8 * (i & 3));
      lw[i >> 2] |= (uint32_t)(q & 0xff) << (8 * (i & 3));
    }
    *reinterpret_cast<uint2*>(xh + (size_t)m * K + (size_t)c * 8) = make_uint2(hw[0], hw[1]);
    *reinterpret_cast<uint2*>(xl + (size_t)m * K + (size_t)c * 8) = make_uint2(lw[0], lw[1]);
  }
}

static int encode_map(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                      const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
  cuuint32_t elem[4] = {1, 1, 1, 1};
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return 999;
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(base), dims,
                                            strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

// Tensor maps are a pure function of (base, extents, box): encoding one costs a driver call of a few
// microseconds, three of them per GEMM would dominate a batched decode step, so they are cached.
struct MapKey {
  const void* base;
  int d0, d1, box;
  bool operator<(const MapKey& o) const { return std::tie(base, d0, d1, box) < std::tie(o.base, o.d0, o.d1, o.box); }
};
// box <= 0: weight map over [n_tiles = d1][KB = d0][8][64] with a box of two k slabs x 16 (box == 0) or -box row tiles,
// 64-byte swizzle; box > 0: limb plane [M = d1][K = d0], box {128, box}, 128-byte swizzle
static int cached_map(CUtensorMap* dst, const void* base, int d0, int d1, int box) {
  static std::map<MapKey, CUtensorMap> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const MapKey key{base, d0, d1, box};
  auto it = cache.find(key);
  if (it == cache.end()) {
    CUtensorMap m;
    int rc;
    if (box <= 0) {
      const cuuint64_t dims[4] = {64, 8, (cuuint64_t)d0, (cuuint64_t)d1};
      const cuuint64_t strides[3] = {64, 512, (cuuint64_t)d0 * 512};
      const cuuint32_t bx[4] = {64, 8, (cuuint32_t)kKS, (cuuint32_t)(box == 0 ? 16 : -box)};
      rc = encode_map(&m, base, 4, dims, strides, bx, CU_TENSOR_MAP_SWIZZLE_64B);
    } else {
      const cuuint64_t dims[2] = {(cuuint64_t)d0, (cuuint64_t)d1};
      const cuuint64_t strides[1] = {(cuuint64_t)d0};
      const cuuint32_t bx[2] = {(cuuint32_t)(kBK * kKS), (cuuint32_t)box};
      rc = encode_map(&m, base, 2, dims, strides, bx, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (rc) return rc;
    if (cache.size() > 8192) cache.clear();
    it = cache.emplace(key, m).first;
  }
  *dst = it->second;
  return 0;
}

template <int BN, bool BF16, int BMH = 1>
static int launch_gemm(const GemmParams& p, dim3 grid, cudaStream_t st) {
  static bool configured = false;
  auto k = gemm_w8a16_kernel<BN, BF16, BMH>;
  if (!configured) {
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GemmGeom<BN, BF16, BMH>::kSmem);
    configured = true;
  }
  const cudaError_t e = launch_kernel(k, grid, dim3(kGemmThreads), GemmGeom<BN, BF16, BMH>::kSmem, st, true, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// 256-row tiles when the token tile is full-size and there are enough tiles to fill the GPU several times over
// (TI_GEMM_BMH=1 / 2 forces a choice)
static int pick_bmh(int M, int n_tiles) {
  static const int forced = [] {
    const char* e = getenv("TI_GEMM_BMH");
    return e == nullptr ? 0 : atoi(e);
  }();
  if (forced == 1 || forced == 2) return n_tiles >= 32 ? forced : 1;
  const long long tiles256 = (long long)((n_tiles * 8 + 255) / 256) * ((M + 127) / 128);
  if (M <= 64) {
    // few tokens: the limb planes are as many bytes per stage as the weights of a 128-row tile; with 256 rows they
    // are half.  That pays only where no k split follows from halving the number of tiles.  Measured at 64 tokens on
    // the 27B shapes (us, 128-row -> 256-row tiles): gate_up 43.6 -> 37.6 (136 tiles, no split), in_proj 23 -> 49
    // (65 tiles in two k slices), down 47 -> 80, out_proj 36 -> 71.  TI_GEMM_BMH_SMALL=1 forces 256 rows.
    static const int small = [] {
      const char* e = getenv("TI_GEMM_BMH_SMALL");
      return e == nullptr ? 0 : atoi(e);
    }();
    if (small && n_tiles >= 64) return 2;
    return tiles256 >= 120 ? 2 : 1;          // enough 256-row tiles to fill the GPU without a k split (gate_up: 44 -> 38 us)
  }
  return (n_tiles >= 32 && tiles256 >= 2 * 148) ? 2 : 1;
}

// k split that fills the 148 SMs when there are few output tiles; sets kb_per_split.  KB counts stages of 128 bytes
// of k; a slice has at least 16 of them (TI_GEMM_SPLIT_STAGES).  Measured at 64 tokens on N = 5120 (us): K = 6144
// unsplit 28.8, three slices 22.2; K = 17408 unsplit 57.5, three slices 32.3.
static int plan_split(GemmParams& p, int KB, int tiles, int M, int N, int ldo, void* part, size_t part_bytes,
                      void* tile_count, int n_count) {
  int S = 1;
  if (part != nullptr && tile_count != nullptr && tiles < 120 && N % 4 == 0 && ldo % 4 == 0) {
    static const int max_split = [] { const char* e = getenv("TI_GEMM_MAX_SPLIT"); return e == nullptr ? 16 : atoi(e); }();
    static const int min_stages = [] { const char* e = getenv("TI_GEMM_SPLIT_STAGES"); return e == nullptr ? 16 : std::max(1, atoi(e)); }();
    S = std::min(std::min(std::min(148 / tiles, KB / min_stages), 16), max_split);
    while (S > 1 && ((size_t)S * M * N * 4 > part_bytes || tiles > n_count)) --S;
    if (S < 1) S = 1;
  }
  p.kb_per_split = (KB + S - 1) / S;
  p.part = (float*)part;
  p.tile_count = (unsigned*)tile_count;
  return (KB + p.kb_per_split - 1) / p.kb_per_split;           // no empty slice
}

}  // namespace ti

extern "C" {

// xh/xl/xscale <- limbs of x (optionally RMS-normalised with (1+norm_w)); one launch, M blocks.
int ti_quant_rows(const void* x, int ldx, const void* norm_w, float eps, int M, int K, void* xh, void* xl, void* xscale,
                  void* stream) {
  if (M <= 0) return 0;
  const bool aligned = (K % 8 == 0) && (ldx % 8 == 0) && (((uintptr_t)x | (uintptr_t)xh | (uintptr_t)xl) % 16 == 0) &&
                       (norm_w == nullptr || (uintptr_t)norm_w % 16 == 0);
  if (aligned && K <= 512 * 5 * 8)
    ti::launch_kernel(ti::quant_rows_fast_kernel, dim3(M), dim3(std::min(512, ((K / 8 + 4) / 5 + 31) / 32 * 32)), 0, (cudaStream_t)stream, true, (const __nv_bfloat16*)x, ldx,
                      (const __nv_bfloat16*)norm_w, eps, K, (int8_t*)xh, (uint8_t*)xl, (float*)xscale);
  else
    ti::quant_rows_kernel<<<M, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)norm_w,
                                                               eps, K, (int8_t*)xh, (uint8_t*)xl, (float*)xscale);
  return (int)cudaGetLastError();
}

// y = x W^T for tiled int8 weights `w` ([n_tiles][K/64][8][64]) and the limb planes of x.
// `part` / `tile_count`: split-k workspace (fp32 [S][M][N]) and zeroed per-tile counters, may be null (no split);
// `part_bytes` / `n_count` are their capacities.  The token tile (32 / 64 / 128) and the k split follow from M, N.
int ti_gemm_w8a16(const void* w, const void* wscale, int n_tiles, int N, int K, const void* xh, const void* xl,
                  const void* xscale, int M, const void* resid, void* out, int ldo, int epi, void* status, void* part,
                  size_t part_bytes, void* tile_count, int n_count, void* stream) {
  if (M <= 0) return 0;
  if (K % 64 || N < 1 || epi < 0 || epi > 2) return -2;
  ti::GemmParams p = {};
  const int KB = K / 64, KS = (KB + ti::kKS - 1) / ti::kKS;      // 64-byte slabs of the weight layout; 128-byte stages
  const int BN = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  const int BMH = ti::pick_bmh(M, n_tiles);
  int rc = ti::cached_map(&p.map_w, w, KB, n_tiles, BMH == 2 ? -32 : 0);
  if (rc) return rc;
  rc = ti::cached_map(&p.map_xh, xh, K, M, BN);
  if (rc) return rc;
  rc = ti::cached_map(&p.map_xl, xl, K, M, BN);
  if (rc) return rc;
  p.xscale = (const float*)xscale;
  p.wscale = (const __nv_bfloat16*)wscale;
  p.resid = (const __nv_bfloat16*)resid;
  p.out = out;
  p.status = (unsigned*)status;
  {
    static const int ablate = [] { const char* e = getenv("TI_GEMM_ABLATE"); return e == nullptr ? 0 : atoi(e); }();
    p.ablate = ablate;
  }
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldo = ldo;
  p.epi = epi;
  const int rows = ti::kBM * BMH;
  const int tiles_n = (n_tiles * 8 + rows - 1) / rows, tiles_m = (M + BN - 1) / BN;
  const int S = ti::plan_split(p, KS, tiles_n * tiles_m, M, N, ldo, part, part_bytes, tile_count, n_count);
  dim3 grid(tiles_m, tiles_n, S);
  cudaStream_t st = (cudaStream_t)stream;
  if (BMH == 2 && BN == 32) return ti::launch_gemm<32, false, 2>(p, grid, st);
  if (BMH == 2 && BN == 64) return ti::launch_gemm<64, false, 2>(p, grid, st);
  if (BMH == 2) return ti::launch_gemm<128, false, 2>(p, grid, st);
  if (BN == 32) return ti::launch_gemm<32, false>(p, grid, st);
  if (BN == 64) return ti::launch_gemm<64, false>(p, grid, st);
  return ti::launch_gemm<128, false>(p, grid, st);
}

// The same for bf16 weights tiled [n_tiles][K/32][8][32] (lm_head, unquantised mode) and bf16 activations x [M][K]
// (contiguous rows): tcgen05.mma kind::f16, fp32 accumulation.  epi 3 stores fp32 (logits).
int ti_gemm_bf16(const void* w, int n_tiles, int N, int K, const void* x, int M, const void* resid, void* out, int ldo,
                 int epi, void* status, void* part, size_t part_bytes, void* tile_count, int n_count, void* stream) {
  if (M <= 0) return 0;
  if (K % 32 || N < 1 || epi < 0 || epi > 3) return -2;
  ti::GemmParams p = {};
  const int KB = K / 32, KS = (KB + ti::kKS - 1) / ti::kKS;    // 64-byte slabs; 128-byte stages
  const int BN = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  const int BMH = ti::pick_bmh(M, n_tiles);
  int rc = ti::cached_map(&p.map_w, w, KB, n_tiles, BMH == 2 ? -32 : 0);
  if (rc) return rc;
  rc = ti::cached_map(&p.map_xh, x, 2 * K, M, BN);
  if (rc) return rc;
  p.resid = (const __nv_bfloat16*)resid;
  p.out = out;
  p.status = (unsigned*)status;
  p.M = M;
  p.N = N;
  p.K = 2 * K;                                                 // bytes of k: the kernel counts 64-byte slabs
  p.ldo = ldo;
  p.epi = epi;
  const int rows = ti::kBM * BMH;
  const int tiles_n = (n_tiles * 8 + rows - 1) / rows, tiles_m = (M + BN - 1) / BN;
  const int S = ti::plan_split(p, KS, tiles_n * tiles_m, M, N, ldo, part, part_bytes, tile_count, n_count);
  dim3 grid(tiles_m, tiles_n, S);
  cudaStream_t st = (cudaStream_t)stream;
  if (BMH == 2 && BN == 32) return ti::launch_gemm<32, true, 2>(p, grid, st);
  if (BMH == 2 && BN == 64) return ti::launch_gemm<64, true, 2>(p, grid, st);
  if (BMH == 2) return ti::launch_gemm<128, true, 2>(p, grid, st);
  if (BN == 32) return ti::launch_gemm<32, true>(p, grid, st);
  if (BN == 64) return ti::launch_gemm<64, true>(p, grid, st);
  return ti::launch_gemm<128, true>(p, grid, st);
}

}  // extern "C"
