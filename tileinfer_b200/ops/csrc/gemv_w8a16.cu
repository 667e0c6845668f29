// Skinny W8A16 / bf16 matrix product for decode: y[M<=16, N] = x[M, K] * W[N, K]^T.
//
// Replaces the reference's dequantize_gemv_kernel (kernels/splitk_gemv.py:131-201), which serves
// M == 1 only with 64-bit weight loads, and its M > 1 fallback that re-materialises a bf16 copy of
// the weight for cuBLAS on every call (kernels/splitk_gemv.py:243-247).
//
// Design for sm_100a:
//  * weights are stored as 512-byte tiles [N/8][K/64][8 rows][64 k] (int8); the tiles of one
//    (row-tile, k-range) unit are contiguous, so every warp streams its units through a private
//    shared-memory ring filled by the TMA engine (cp.async.bulk + mbarrier, 2 KB stages): up to
//    ~190 KB of weights are in flight per SM without holding registers, which is what it takes to
//    cover HBM latency at 6.5 TB/s; a lane then reads its 128-bit slice of a tile conflict-free;
//  * int8 weights are never widened.  The bf16 activations of a row are split exactly into two int8
//    limbs of a 16-bit fixed-point number with one power-of-two exponent per row (x = (256 hi + lo)
//    2^(e-14), hi signed, lo unsigned), staged once per CTA in shared memory, and both limbs are
//    multiplied with the raw int8 weights on the integer tensor cores (mma.sync.m16n8k32 s8 x s8 and
//    u8 x s8, int32 accumulation, so the dot product itself is exact): 4 MMAs and 3 shared-memory loads
//    per 512-byte weight tile instead of ~44 conversion instructions.  Activations are the 16-row A
//    operand (one weight pass serves up to 16 tokens), the 8 weight rows of the tile are the B operand;
//    bf16 weights (lm_head, unquantised mode) use mma.sync.m16n8k16 bf16 with fp32 accumulation;
//  * work is split into (row-tile, k-range) units spread over all warps of a persistent grid;
//    split-k partials meet in a workspace and the last warp to arrive sums them in a fixed order
//    (deterministic) and runs the epilogue;
//  * prologue fusion: RMSNorm(1+w) of the residual stream is applied while staging x in shared
//    memory (replaces kernels/rms_norm.py and the norm half of kernels/residual_rmsnorm.py);
//  * epilogue fusion: bf16 store, SwiGLU (kernels/act_mul.py), fp32 logits, or the row-parallel
//    epilogue: the per-rank partial is pushed as tagged 8-byte packets straight into every peer's
//    buffer over NVLink, the packets of the other ranks are awaited (bounded), summed in rank
//    order and added to the residual (replaces the NCCL all-reduce + residual add of
//    model/qwen_36.py:759-771, 795-803, 1088-1095, 1119-1127).
#include <algorithm>
#include "common.cuh"

namespace ti {

struct GemvParams {
  const uint8_t* w;              // tiled weights
  const __nv_bfloat16* scale;    // [n_pad] per-row scale (int8) or nullptr (bf16 weights)
  const __nv_bfloat16* x;        // XGLOBAL: activations [M, ldx]; XNORM: residual stream [M, K]
  const __nv_bfloat16* norm_w;   // XNORM: RMSNorm weight (1+w convention) [K]
  void* out;                     // see epilogues
  const __nv_bfloat16* resid;    // ROWPAR: residual in [M, N]
  float* ws;                     // split-k partials [units][128]
  unsigned* counters;            // [n_tiles], zero between launches
  const unsigned* step_ptr;      // device step counter (tag source), ROWPAR with tp > 1
  unsigned* status;              // error bits
  uint64_t peer_ll[kMaxRanks];   // packet buffers of all ranks as mapped in this process
  unsigned long long timeout_ns;
  int M, N, n_tiles, K, KB, S, kb_per_split;
  int ldx, ldo;
  int tp, rank, order, m_cap;
  float eps;
  int stages;                    // depth of the per-warp weight ring (1..8)
  int T;                         // team size (1..16 adjacent warps of a CTA share a unit, each a k-slice)
  unsigned long long* dbg;       // optional [ncta][32] globaltimer stamps of warp 0 (profiling aid): 0 start, 1 ring
                                 // primed, 2..4 all warps of the CTA reached the barrier before product 1..3, 5 end; per product op at 8 + 4*op:
                                 // marker reached, barrier passed, x staged, last unit done
  int* sched;                    // dynamic scheduling state: [0] launches finished, [1] CTAs finished, [8 + 3*16] tickets
  int tps;                       // 512-byte tiles per ring stage (4, 8 or 16)
  int xmode, epi;                // XGLOBAL | XNORM ; EPI_*
  int R;                         // row tiles (of 8 weight rows) per unit: 1 or 2
  int xll;                       // 1: x is the all-reduced output of the PREVIOUS product of the chain (row-parallel, tp > 1);
                                 // every CTA collects that product's packets itself instead of waiting for a collect pass
                                 // and a grid barrier
  int* out_idx;                  // EPI_ARGMAX: [M][ncta] column of each CTA's candidate (`out`: float [M][ncta] values)
};

// Up to four dependent products run back to back in one launch (e.g. out_proj -> gate_up -> down -> the
// next layer's in_proj): a grid barrier separates them, the weight streams of the warps run ahead into the
// next product while the barrier and the activation staging take place, so HBM never drains between them.
constexpr int kMaxChain = 4;
struct ChainParams {
  int n_ops;
  int x_bytes;                   // shared memory reserved for staged activations (max over the ops)
  GemvParams op[kMaxChain];
};

// Shared-memory footprint of the staged activations (+ 2 KB of reduction scratch).
//   bf16 weights: rows(8|16) x (K+8) bf16          int8 weights: two limb planes of M x stride bytes
TI_HOST_DEVICE int limb_stride(int kslice) { return kslice + ((64 - (kslice % 128)) + 128) % 128; }
TI_HOST_DEVICE size_t x_smem_bytes_impl(int wt, int xmode, int M, int K, int kslice) {
  size_t b = 0;
  if (wt == 0) b = (size_t)2 * M * limb_stride(kslice);
  else if (xmode == 1) b = (size_t)(M > 8 ? 16 : 8) * (K + 8) * 2;
  return (b + 2048 + 127) / 128 * 128;
}

enum { XGLOBAL = 0, XNORM = 1 };
// EPI_ARGMAX: nothing is stored per output; every warp keeps the best (value, column) of each activation row over the
// row tiles it owns, the CTA reduces them, and writes ONE candidate per row and CTA to out / out_idx ([M][gridDim]):
// the lm_head product fused with the first stage of the arg-max (greedy sampling needs no logits in memory).
enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_ROWPAR = 2, EPI_F32 = 3, EPI_ARGMAX = 4 };
enum { W_INT8 = 0, W_BF16 = 1 };

#ifndef TI_GEMV_WARPS
#define TI_GEMV_WARPS 16
#endif
constexpr int kThreads = TI_GEMV_WARPS * 32;
#ifndef TI_GEMV_TPS
#define TI_GEMV_TPS 8
#endif
constexpr int kTPS = TI_GEMV_TPS;          // 512-byte tiles per ring stage (8: 4 KB)
constexpr int kMaxStages = 16;
constexpr int kMaxTilesPerStage = 16;
constexpr int kWarps = kThreads / 32;
constexpr int kCQ = 16;                    // per-warp queue of scheduled units
constexpr int kLook = 1;                   // entries a warp queues ahead of its consumer side.  Kept small on purpose: a warp
                                           // that draws tickets far ahead (or one ticket in advance) hoards units of a product
                                           // while it is still idle or busy elsewhere, and the product then ends on the few
                                           // warps that hold three or four units each
constexpr int kMaxR = 4;                   // row tiles per unit
constexpr int kTeamBytes = 2 * kWarps * 32 * 16;   // team-mode exchange buffer

// Operands of the epilogue that do not depend on the product: fetched when a warp STARTS a row tile, so that
// their latency (an L2 round trip for the residual) is not paid after the last tile, where in team mode the whole
// team would wait for it.
struct EpiPre { float s0, s1; uint32_t r0, r1; };
TI_DEVICE EpiPre epi_prefetch(const GemvParams& p, int nt, int g, int t) {
  EpiPre e{1.f, 1.f, 0u, 0u};
  const int n = nt * 8 + 2 * t;
  if (n >= p.N) return e;
  if (p.scale != nullptr) {
    e.s0 = bf16_to_f(p.scale[n]);
    e.s1 = bf16_to_f(p.scale[n + 1]);
  }
  if (p.epi == EPI_ROWPAR && p.tp == 1) {
    if (g < p.M) e.r0 = __ldcg(reinterpret_cast<const uint32_t*>(p.resid + (size_t)g * p.N + n));
    if (g + 8 < p.M) e.r1 = __ldcg(reinterpret_cast<const uint32_t*>(p.resid + (size_t)(g + 8) * p.N + n));
  }
  return e;
}

TI_DEVICE void epilogue(const GemvParams& p, int nt, int g, int t, const float (&acc)[4], const EpiPre& pre) {
  const int n = nt * 8 + 2 * t;
  if (n >= p.N) return;
  const float s0 = pre.s0, s1 = pre.s1;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = g + half * 8;
    if (m >= p.M) continue;
    float v0 = acc[half * 2] * s0, v1 = acc[half * 2 + 1] * s1;
    if (p.epi == EPI_STORE) {
      uint32_t* o = reinterpret_cast<uint32_t*>(static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldo + n);
      *o = pack_bf16(v0, v1);
    } else if (p.epi == EPI_F32) {
      float2* o = reinterpret_cast<float2*>(static_cast<float*>(p.out) + (size_t)m * p.ldo + n);
      *o = make_float2(v0, v1);
    } else if (p.epi == EPI_SWIGLU) {
      // rows come interleaved (gate, up); both are rounded to bf16 first, as a separate activation
      // kernel reading bf16 projections would see them
      const float gate = round_bf16(v0), up = round_bf16(v1);
      static_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + (n >> 1)] = __float2bfloat16_rn(silu_f(gate) * up);
    } else {  // EPI_ROWPAR
      if (p.tp > 1) {
        // Send only: the partial goes, tagged, into the packet buffer of EVERY rank (this one included).
        // Nothing is awaited here, so ranks whose warps take the row tiles in a different order can never
        // wait on each other in a cycle; rowpar_reduce() collects the packets once the product is done.
        const unsigned tag = (*p.step_ptr) * 65536u + (unsigned)p.order + 1u;
        const int slot = p.order & 1;
        const size_t mine = ((((size_t)slot * p.tp + p.rank) * p.m_cap + m) * (size_t)(p.N >> 1) + (n >> 1)) * 16;
        jitter();
        if (TI_CHECK(mine + 15, (size_t)2 * p.tp * p.m_cap * (size_t)(p.N >> 1) * 16, p.status))
          for (int q = 0; q < p.tp; ++q) ll_store2(reinterpret_cast<uint8_t*>(p.peer_ll[q]) + mine, v0, v1, tag);
      } else {
        const uint32_t rw = half ? pre.r1 : pre.r0;
        uint32_t* o = reinterpret_cast<uint32_t*>(static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.N + n);
        *o = pack_bf16(bf16lo(rw) + v0, bf16hi(rw) + v1);
      }
    }
  }
}

// Second half of the fused all-reduce of a row-parallel product (tp > 1): every thread of the grid takes
// some (row, column pair) positions, waits (bounded) for the tagged packets of all ranks, adds them in rank
// order (so every rank computes bit-identical sums) and adds the residual.
// (cta, ncta) = (blockIdx, gridDim): the grid shares the positions; (0, 1): this CTA takes all of them (every CTA
// of the grid then writes the same values: the consumer is the next product's staging in the same CTA).
TI_DEVICE void rowpar_reduce(const GemvParams& p, int cta, int ncta) {
  const unsigned tag = (*p.step_ptr) * 65536u + (unsigned)p.order + 1u;
  const int slot = p.order & 1;
  const int pairs = p.N >> 1;
  const uint8_t* local = reinterpret_cast<const uint8_t*>(p.peer_ll[p.rank]);
  jitter();
  for (int i = cta * blockDim.x + threadIdx.x; i < p.M * pairs; i += ncta * blockDim.x) {
    const int m = i / pairs, pr = i - m * pairs;
    float s0 = 0.f, s1 = 0.f;
    for (int r = 0; r < p.tp; ++r) {
      float a = 0.f, b = 0.f;
      const size_t off = ((((size_t)slot * p.tp + r) * p.m_cap + m) * (size_t)pairs + pr) * 16;
      if (TI_CHECK(off + 15, (size_t)2 * p.tp * p.m_cap * (size_t)pairs * 16, p.status))
        ll_wait2(local + off, tag, a, b, p.timeout_ns, p.status);
      s0 += a;
      s1 += b;
    }
    const uint32_t rw = __ldcg(reinterpret_cast<const uint32_t*>(p.resid + (size_t)m * p.N + 2 * pr));
    uint32_t* o = reinterpret_cast<uint32_t*>(static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.N + 2 * pr);
    *o = pack_bf16(bf16lo(rw) + s0, bf16hi(rw) + s1);
  }
}

// Activations may have been written earlier in the SAME launch by another SM (chained products): read them
// through L2, never through the non-coherent path.
TI_DEVICE uint4 ld_x16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

TI_DEVICE uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// ---------------------------------------------------------------- integer tensor-core MMAs
TI_DEVICE void imma_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
TI_DEVICE void imma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------- activation staging
// Per-row statistics scratch: red[nwarps][16] then rowv[16] (rrms), rows[16] (limb scale 2^(e-14)).
TI_DEVICE void block_row_reduce(float (&v)[16], int M, float* red, float* out, int tid, bool is_max) {
  const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  for (int m = 0; m < M; ++m) {
    const float r = is_max ? warp_max(v[m]) : warp_sum(v[m]);
    if (lane == 0) red[warp * 16 + m] = r;
  }
  __syncthreads();
  if (tid < M) {
    float a = is_max ? 0.f : 0.f;
    for (int w = 0; w < nwarps; ++w) a = is_max ? fmaxf(a, red[w * 16 + tid]) : a + red[w * 16 + tid];
    out[tid] = a;
  }
  __syncthreads();
}

// Stages the k-slice [k_lo, k_hi) of up to 16 rows as two int8 limb planes.  XNORM: the rows are first
// RMS-normalised with (1+w) (statistics over the full row) and rounded to bf16.
TI_DEVICE void stage_limbs(const GemvParams& p, int k_lo, int k_hi, int8_t* xh, uint8_t* xl, int stride, float* scratch) {
  const int tid = threadIdx.x;
  float* red = scratch;            // [16 warps][16]
  float* rrms = scratch + 256;     // [16]
  float* amax = scratch + 272;     // [16]
  float* inv = scratch + 288;      // [16]  2^(e-14): value of one fixed-point unit
  const int nthreads = blockDim.x;
  // ---- single-row fast path (batch-1 decode): the row lives in registers, read from memory once
  if (p.M == 1 && (k_hi - k_lo) <= 40 * nthreads && (p.xmode != XNORM || (k_lo == 0 && k_hi == p.K))) {
    const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
    const int c_lo = k_lo >> 3, c_hi = k_hi >> 3;
    float v[5][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 5; ++j) {
      const int c = c_lo + tid + j * nthreads;
      uint4 q = make_uint4(0, 0, 0, 0);
      if (c < c_hi) q = ld_x16(p.x + (size_t)c * 8);
      const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[j][2 * i] = bf16lo(w4[i]);
        v[j][2 * i + 1] = bf16hi(w4[i]);
        ss += v[j][2 * i] * v[j][2 * i] + v[j][2 * i + 1] * v[j][2 * i + 1];
      }
    }
    if (p.xmode == XNORM) {
      // the norm weights do not depend on x: their loads are in flight together with those of x
      uint4 nwv[5];
#pragma unroll
      for (int j = 0; j < 5; ++j) {
        const int c = c_lo + tid + j * nthreads;
        nwv[j] = c < c_hi ? ldg_cached16(p.norm_w + (size_t)c * 8) : make_uint4(0, 0, 0, 0);
      }
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < nwarps; ++w) tot += red[w];
      const float rr = rsqrtf(tot / (float)p.K + p.eps);
#pragma unroll
      for (int j = 0; j < 5; ++j) {
        const int c = c_lo + tid + j * nthreads;
        if (c >= c_hi) continue;
        const uint4 nw = nwv[j];
        const uint32_t n4[4] = {nw.x, nw.y, nw.z, nw.w};
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
    if (lane == 0) red[32 + warp] = mx;
    __syncthreads();
    float a = 0.f;
    for (int w = 0; w < nwarps; ++w) a = fmaxf(a, red[32 + w]);
    int e = (int)((__float_as_uint(a) >> 23) & 0xffu) - 127;
    e = max(e, -100);
    if (!(a < 3.0e38f)) e = 127;
    const float qs = exp2f((float)(14 - e));
    if (tid == 0) inv[0] = exp2f((float)(e - 14));
#pragma unroll
    for (int j = 0; j < 5; ++j) {
      const int c = c_lo + tid + j * nthreads;
      if (c >= c_hi) continue;
      uint32_t hw[2] = {0, 0}, lw[2] = {0, 0};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int q = max(-32768, min(32767, __float2int_rn(v[j][i] * qs)));
        hw[i >> 2] |= (uint32_t)((q >> 8) & 0xff) << (8 * (i & 3));
        lw[i >> 2] |= (uint32_t)(q & 0xff) << (8 * (i & 3));
      }
      const size_t o = (size_t)(c - c_lo) * 8;
      *reinterpret_cast<uint2*>(xh + o) = make_uint2(hw[0], hw[1]);
      *reinterpret_cast<uint2*>(xl + o) = make_uint2(lw[0], lw[1]);
    }
    __syncthreads();
    return;
  }
  float acc[16];
  if (p.xmode == XNORM) {
#pragma unroll
    for (int m = 0; m < 16; ++m) acc[m] = 0.f;
    for (int c = tid; c < (p.K >> 3); c += blockDim.x) {
#pragma unroll
      for (int m = 0; m < 16; ++m) {
        if (m >= p.M) break;
        const uint4 v = ld_x16(p.x + (size_t)m * p.ldx + c * 8);
        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m] += bf16lo(w4[i]) * bf16lo(w4[i]) + bf16hi(w4[i]) * bf16hi(w4[i]);
      }
    }
    block_row_reduce(acc, p.M, red, rrms, tid, false);
    if (tid < p.M) rrms[tid] = rsqrtf(rrms[tid] / (float)p.K + p.eps);
    __syncthreads();
  }
  // pass A: row maxima over the slice
#pragma unroll
  for (int m = 0; m < 16; ++m) acc[m] = 0.f;
  const int c_lo = k_lo >> 3, c_hi = k_hi >> 3;
  for (int c = c_lo + tid; c < c_hi; c += blockDim.x) {
    uint4 nw = make_uint4(0, 0, 0, 0);
    if (p.xmode == XNORM) nw = ldg_cached16(p.norm_w + c * 8);
    const uint32_t n4[4] = {nw.x, nw.y, nw.z, nw.w};
#pragma unroll
    for (int m = 0; m < 16; ++m) {
      if (m >= p.M) break;
      const uint4 v = ld_x16(p.x + (size_t)m * p.ldx + c * 8);
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
      const float rr = p.xmode == XNORM ? rrms[m] : 1.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float a = bf16lo(w4[i]), b = bf16hi(w4[i]);
        if (p.xmode == XNORM) {
          a = round_bf16(a * rr * (1.f + bf16lo(n4[i])));
          b = round_bf16(b * rr * (1.f + bf16hi(n4[i])));
        }
        acc[m] = fmaxf(acc[m], fmaxf(fabsf(a), fabsf(b)));
      }
    }
  }
  block_row_reduce(acc, p.M, red, amax, tid, true);
  if (tid < p.M) {
    const float a = amax[tid];
    int e = (int)((__float_as_uint(a) >> 23) & 0xffu) - 127;
    e = max(e, -100);
    if (!(a < 3.0e38f)) e = 127;                 // inf / nan rows: keep finite arithmetic
    amax[tid] = exp2f((float)(14 - e));          // quantisation scale
    inv[tid] = exp2f((float)(e - 14));
  }
  __syncthreads();
  // pass B: quantise and store the limb planes
  for (int c = c_lo + tid; c < c_hi; c += blockDim.x) {
    uint4 nw = make_uint4(0, 0, 0, 0);
    if (p.xmode == XNORM) nw = ldg_cached16(p.norm_w + c * 8);
    const uint32_t n4[4] = {nw.x, nw.y, nw.z, nw.w};
#pragma unroll
    for (int m = 0; m < 16; ++m) {
      if (m >= p.M) break;
      const uint4 v = ld_x16(p.x + (size_t)m * p.ldx + c * 8);
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
      const float rr = p.xmode == XNORM ? rrms[m] : 1.f, qs = amax[m];
      uint32_t hw[2] = {0, 0}, lw[2] = {0, 0};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float a = bf16lo(w4[i]), b = bf16hi(w4[i]);
        if (p.xmode == XNORM) {
          a = round_bf16(a * rr * (1.f + bf16lo(n4[i])));
          b = round_bf16(b * rr * (1.f + bf16hi(n4[i])));
        }
        const int qa = max(-32768, min(32767, __float2int_rn(a * qs)));
        const int qb = max(-32768, min(32767, __float2int_rn(b * qs)));
        const int e0 = 2 * i, e1 = 2 * i + 1;
        hw[e0 >> 2] |= (uint32_t)((qa >> 8) & 0xff) << (8 * (e0 & 3));
        hw[e1 >> 2] |= (uint32_t)((qb >> 8) & 0xff) << (8 * (e1 & 3));
        lw[e0 >> 2] |= (uint32_t)(qa & 0xff) << (8 * (e0 & 3));
        lw[e1 >> 2] |= (uint32_t)(qb & 0xff) << (8 * (e1 & 3));
      }
      const size_t o = (size_t)m * stride + (size_t)(c - c_lo) * 8;
      *reinterpret_cast<uint2*>(xh + o) = make_uint2(hw[0], hw[1]);
      *reinterpret_cast<uint2*>(xl + o) = make_uint2(lw[0], lw[1]);
    }
  }
  __syncthreads();
}

// bf16-weight path: RMSNorm(1+w) of up to 16 rows into shared memory as bf16.
TI_DEVICE void stage_bf16_norm(const GemvParams& p, __nv_bfloat16* xs, int xs_stride, float* scratch) {
  const int tid = threadIdx.x;
  const int rows = p.M > 8 ? 16 : 8;
  float* red = scratch;
  float* rrms = scratch + 256;
  float acc[16];
#pragma unroll
  for (int m = 0; m < 16; ++m) acc[m] = 0.f;
  const int chunks = p.K >> 3;
  for (int c = tid; c < chunks; c += blockDim.x) {
#pragma unroll
    for (int m = 0; m < 16; ++m) {
      if (m >= p.M) break;
      const uint4 v = ld_x16(p.x + (size_t)m * p.ldx + c * 8);
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m] += bf16lo(w4[i]) * bf16lo(w4[i]) + bf16hi(w4[i]) * bf16hi(w4[i]);
    }
  }
  block_row_reduce(acc, p.M, red, rrms, tid, false);
  if (tid < p.M) rrms[tid] = rsqrtf(rrms[tid] / (float)p.K + p.eps);
  __syncthreads();
  for (int c = tid; c < chunks; c += blockDim.x) {
    const uint4 nw = ldg_cached16(p.norm_w + c * 8);
    const uint32_t n4[4] = {nw.x, nw.y, nw.z, nw.w};
    for (int m = 0; m < rows; ++m) {
      uint4 o = make_uint4(0, 0, 0, 0);
      if (m < p.M) {
        const uint4 v = ld_x16(p.x + (size_t)m * p.ldx + c * 8);
        const uint32_t a4[4] = {v.x, v.y, v.z, v.w};
        const float rr = rrms[m];
        uint32_t r4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          r4[i] = pack_bf16(bf16lo(a4[i]) * rr * (1.f + bf16lo(n4[i])), bf16hi(a4[i]) * rr * (1.f + bf16hi(n4[i])));
        o = make_uint4(r4[0], r4[1], r4[2], r4[3]);
      }
      *reinterpret_cast<uint4*>(xs + (size_t)m * xs_stride + c * 8) = o;
    }
  }
  __syncthreads();
}

// ---------------------------------------------------------------- work decomposition
// A unit is R consecutive row tiles (8 weight rows each) over the WHOLE k range, owned by ONE warp: no
// partial sum ever leaves the warp, nothing is reduced, fenced or counted anywhere.  A warp streams its
// unit through a private ring of shared memory filled by TMA bulk copies (the tiles of a row tile are
// contiguous), deep enough to cover HBM latency at that warp's share of the bandwidth, and keeps
// streaming across units and across the products of a chain.  Units are dealt to warps: the first ones
// statically (spread over the SMs first), the rest through one ticket counter per product, drawn when
// the copy side runs out of work.  A per-warp queue in shared memory carries the unit sequence from the issuing side (lane 0
// runs ahead with the copies) to the consuming side.
// Products with few row tiles (N = 5120: 640 row tiles for 2368 warps) would leave most warps, and with them
// most of the bytes in flight, idle.  They run in team mode instead (T > 1): the T warps of a team (same CTA,
// adjacent warp ids) share a unit, each streams its own slice of the k range, the partial sums meet in shared
// memory behind a named barrier and the first warp of the team adds them in slice order and runs the epilogue.
// Team units are dealt statically, unit u to team u mod (number of teams).
TI_DEVICE int num_units(const GemvParams& p) { return (p.n_tiles + p.R - 1) / p.R; }
#define TI_UNIT_END (-1)
constexpr int kUnitMask = (1 << 26) - 1;
TI_DEVICE int pack_unit(int op, int unit) { return (op << 26) | unit; }
// queue entry that opens product `op`: every warp sees it (and takes part in the grid barrier and the
// activation staging of that product) whether or not it gets any unit of the product
TI_DEVICE int pack_begin(int op) { return (op << 26) | kUnitMask; }
// Units k*W + widx for k < ns are assigned statically (no atomics: they can be queued before the kernel may
// look at mutable state); the rest of a product's units go through the ticket counter, which evens out warps
// that fell behind.
// Per-warp, per-product scheduling constants, worked out once at kernel start (they hold integer divisions that
// would otherwise be redone by lane 0 for every unit, with the other lanes of the warp and the warp's issue slots
// waiting; with the short units of tensor-parallel shards that was a third of a product's time).
enum { TB_U = 0, TB_WD, TB_NS, TB_WIDX, TB_MEMBER, TB_BASE, TB_REM, TB_T, TB_N };
TI_DEVICE void fill_op_table(const ChainParams& c, int warp, int cta, int ncta, int* tb) {
  const int W = ncta * kWarps, widx = warp * ncta + cta;
  for (int op = 0; op < c.n_ops; ++op) {
    const GemvParams& p = c.op[op];
    const int U = num_units(p), T = p.T;
    // team mode: a CTA holds kWarps / T whole teams (any T up to kWarps; the warps left over when T does not
    // divide kWarps take no unit of this product)
    const int tpc = kWarps / T;
    const int Wd = T > 1 ? tpc * ncta : W;
    const bool active = T == 1 || warp < tpc * T;
    int* t = tb + op * TB_N;
    t[TB_U] = active ? U : 0;
    t[TB_WD] = Wd;
    t[TB_NS] = !active ? 0 : (T > 1 ? (U + Wd - 1) / Wd : max(1, U / (2 * W)));
    t[TB_WIDX] = T > 1 ? (warp / T) * ncta + cta : widx;
    t[TB_MEMBER] = T > 1 ? warp % T : 0;
    t[TB_BASE] = p.KB / T;
    t[TB_REM] = p.KB - (p.KB / T) * T;
    t[TB_T] = T;
  }
}
// k-slice [kt0, kt0 + run) of this warp in product `op` (the whole k range outside team mode)
TI_DEVICE void my_slice(const int* tb, int op, int& kt0, int& run) {
  const int* t = tb + op * TB_N;
  const int j = t[TB_MEMBER], base = t[TB_BASE], rem = t[TB_REM];
  kt0 = j * base + min(j, rem);
  run = base + (j < rem ? 1 : 0);
}

struct WarpStream {           // registers of lane 0 of each warp; queue storage in shared memory
  const int* tb;              // this warp's table of scheduling constants
  // scheduling side
  int op, sk, wr, rd;
  bool sdone, can_ticket, opened;
  // copy side
  int cs, idx, left, row_left, kb_row;
  uint32_t ist, skip;
  bool have, cdone;
  const uint8_t* gptr;

  TI_DEVICE void push(volatile int* q, int e) { q[wr++ % kCQ] = e; }
  // queue the next entries of this warp's unit sequence, at most up to `ahead` entries beyond `rd`
  TI_DEVICE void schedule(const ChainParams& c, int widx, int W, volatile int* q, int ahead) {
    while (!sdone && wr - rd < kCQ - 2) {
      const GemvParams& p = c.op[op];
      // team mode: the "worker" is the team, and every unit is static
      const int* t = tb + op * TB_N;
      const int U = t[TB_U], Wd = t[TB_WD], wd = t[TB_WIDX], ns = t[TB_NS];
      if (!opened) {
        opened = true;
        push(q, pack_begin(op));
        continue;
      }
      if (sk < ns) {
        // static units take from nobody: they may be queued further ahead than tickets (matters for the small
        // units of team mode, where the ring holds more than one unit)
        const int u = sk * Wd + wd;
        ++sk;
        if (u < U) push(q, pack_unit(op, u));
        continue;
      }
      if (!can_ticket || wr - rd >= ahead) return;
      // drawn only when the copy side has handed the whole previous unit to the TMA engine: the consumer side
      // is then still a ring's depth of chunks behind, which covers the latency of the atomic
      // (no draw at all when the static deal already covers the product: 2368 warps hitting one counter at
      // the end of every small product cost microseconds)
      const int u = (t[TB_T] > 1 || ns * W >= U) ? U : ns * W + atomicAdd(p.sched + 8 + op * 16, 1);
      if (u >= U) {
        sk = 0;
        opened = false;
        if (++op >= c.n_ops) {
          push(q, TI_UNIT_END);
          sdone = true;
        }
        continue;
      }
      push(q, pack_unit(op, u));
    }
  }
  TI_DEVICE bool load(const ChainParams& c, int widx, int W, volatile int* q) {
    while (!cdone) {
      if (cs >= wr) schedule(c, widx, W, q, kLook);
      if (cs >= wr) return false;
      const int e = q[cs % kCQ];
      if (e == TI_UNIT_END) {
        cdone = true;
        return false;
      }
      const int unit = e & kUnitMask;
      if (unit == kUnitMask) {             // product marker: nothing to stream
        ++cs;
        continue;
      }
      const GemvParams& p = c.op[e >> 26];
      // one run of tiles per row tile of the unit; outside team mode the runs are adjacent in memory
      const int grp = unit;
      int kt0, run;
      my_slice(tb, e >> 26, kt0, run);
      const int rn = min(p.R, p.n_tiles - grp * p.R);
      left = rn * run;
      row_left = run;
      kb_row = run;
      skip = (uint32_t)(p.KB - run) * 512u;
      gptr = p.w + ((size_t)grp * p.R * p.KB + kt0) * 512;
      have = true;
      return true;
    }
    return false;
  }
  // hands the next chunk (<= kTPS tiles, never across a row tile) to the TMA engine
  TI_DEVICE void next(const ChainParams& c, int widx, int W, volatile int* q, uint32_t ring_u32, uint32_t bar0,
                      int stages) {
    if (!have && !load(c, widx, W, q)) return;
    const int ntile = min(kTPS, row_left);
    const uint32_t bytes = (uint32_t)ntile * 512u;
    mbar_expect_tx(bar0 + ist * 8, bytes);
    bulk_g2s(ring_u32 + ist * (kTPS * 512u), gptr, bytes, bar0 + ist * 8);
    ist = ist + 1 == (uint32_t)stages ? 0u : ist + 1;
    ++idx;
    gptr += bytes;
    left -= ntile;
    row_left -= ntile;
    if (row_left == 0) {
      row_left = kb_row;
      gptr += skip;
    }
    if (left == 0) {
      have = false;
      ++cs;
    }
  }
};

// Optional (-DTI_GEMV_PREFETCH_KB=n, off by default): while the previous kernel of the stream is still running
// (before griddepcontrol.wait) the rings hold only a few stages per warp; what follows them in this warp's first unit
// of the first two products can be asked into L2.  Measured with 24 KB per warp on the 27B layer: the chain alone
// 87.5 -> 90.5 us and the decode step 6.70 -> 7.0 ms: the prefetches compete with the ring fills of all warps for the
// same HBM queue at the moment the chain starts, so it stays off.
#ifndef TI_GEMV_PREFETCH_KB
#define TI_GEMV_PREFETCH_KB 0
#endif
TI_DEVICE void l2_prefetch(const void* ptr, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(ptr), "r"(bytes) : "memory");
}
TI_DEVICE void prefetch_ahead(const ChainParams& c, const int* tb, int stages) {
  int budget = TI_GEMV_PREFETCH_KB * 1024;
  int skip = stages * kTPS * 512;                      // already requested through the ring
  for (int op = 0; op < c.n_ops && op < 2 && budget > 0; ++op) {
    const int* t = tb + op * TB_N;
    const GemvParams& p = c.op[op];
    const int u = t[TB_WIDX];
    if (t[TB_NS] >= 1 && u < t[TB_U]) {
      int kt0, run;
      my_slice(tb, op, kt0, run);
      const int rn = min(p.R, p.n_tiles - u * p.R);
      for (int r = 0; r < rn && budget > 0; ++r) {
        const uint8_t* base = p.w + ((size_t)(u * p.R + r) * p.KB + kt0) * 512;
        const int bytes = run * 512;
        const int off = min(skip, bytes);
        skip -= off;
        const int n = min(bytes - off, budget);
        if (n > 0) {
          l2_prefetch(base + off, (uint32_t)n);
          budget -= n;
        }
      }
    }
    skip = 0;
  }
}

// Grid-wide barrier between chained products.  All CTAs of the launch are resident (one per SM), the
// counter is reset by the last CTA of the launch.  The wait is bounded like every other wait here.
TI_DEVICE void grid_barrier(int* counter, int target, unsigned* status, unsigned long long* arrived = nullptr) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (arrived != nullptr) *arrived = globaltimer_ns();   // every warp of this CTA is done with the product
    __threadfence();
    atomicAdd(counter, 1);
    const unsigned long long t0 = globaltimer_ns();
    unsigned spins = 0;
    while (true) {
      int v;
      asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(counter) : "memory");
      if (v >= target) break;
      if ((++spins & 63u) == 0u && globaltimer_ns() - t0 > 2000000000ull) {
        if (status != nullptr) atomicOr(status, kStatusPeerTimeout);
        break;
      }
    }
    __threadfence();
  }
  __syncthreads();
}

// ---------------------------------------------------------------- main body
template <int WT>
TI_DEVICE void gemv_body(const ChainParams& c, int cta, int ncta, uint8_t* smem) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const GemvParams& p0 = c.op[0];
  const bool stamp = p0.dbg != nullptr && tid == 0;
  if (stamp) p0.dbg[cta * 32 + 0] = globaltimer_ns();
  const size_t x_bytes = (size_t)c.x_bytes;
  const int W = ncta * kWarps, widx = warp * ncta + cta;      // consecutive units land on different SMs

  // ---- shared memory: [staged x | rings | mbarriers | unit queues]
  const int stages = p0.stages;
  const int stage_bytes = kTPS * 512;
  uint8_t* ring0 = smem + x_bytes;
  uint8_t* ring = ring0 + (size_t)warp * stages * stage_bytes;
  const uint32_t ring_u32 = smem_u32(ring);
  uint8_t* after_ring = ring0 + (size_t)kWarps * stages * stage_bytes;
  const uint32_t bar0 = smem_u32(after_ring) + warp * stages * 8;
  volatile int* q = reinterpret_cast<volatile int*>(after_ring + kWarps * stages * 8) + warp * kCQ;
  float4* tscr = reinterpret_cast<float4*>(after_ring + kWarps * (stages * 8 + kCQ * 4));   // [2][kWarps][32], team mode

  __shared__ int optab[kWarps][kMaxChain * TB_N];
  int* tb = optab[warp];
  if (lane == 0) fill_op_table(c, warp, cta, ncta, tb);
  __syncwarp();
  WarpStream ws;
  ws.tb = tb;
  ws.op = ws.sk = ws.wr = ws.rd = 0;
  ws.sdone = ws.can_ticket = ws.opened = false;
  ws.cs = ws.idx = ws.left = ws.row_left = ws.kb_row = 0;
  ws.ist = ws.skip = 0;
  ws.have = ws.cdone = false;
  ws.gptr = nullptr;
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(bar0 + s * 8, 1);
    fence_mbar_init();
    for (int s = 0; s < stages; ++s) ws.next(c, widx, W, q, ring_u32, bar0, stages);   // static units only
    if (TI_GEMV_PREFETCH_KB > 0) prefetch_ahead(c, tb, stages);
  }
  __syncwarp();
  // Everything above touched only weights and this CTA's shared memory.  Let the next kernel of the
  // stream start its own prefetch, then wait until the previous kernel (which produced x and may still
  // be using the tickets) has completed.
  pdl_trigger();
  pdl_wait();
  if (stamp) p0.dbg[cta * 32 + 1] = globaltimer_ns();
  if (lane == 0) ws.can_ticket = true;

  // EPI_ARGMAX: best (value, column) seen by this lane for rows g and g + 8 over all the row tiles of its warp
  float am_v0 = -INFINITY, am_v1 = -INFINITY;
  int am_i0 = 0x7fffffff, am_i1 = 0x7fffffff;
  unsigned cidx = 0;                            // chunks consumed by this warp so far
  uint32_t cst = 0, cpar = 0;                   // ring stage / mbarrier phase of the next chunk to consume
  unsigned tcount = 0;                          // team exchanges of this warp in the current product
  int cur_op = -1, nbar = 0;                    // nbar: grid barriers passed (the same sequence in every CTA)
  bool alive = true;
  float* scratch = reinterpret_cast<float*>(smem + x_bytes - 2048);
  float inv0 = 0.f, inv1 = 0.f;                 // value of one fixed-point unit for rows g and g+8
  int lstride = 0;
  int8_t* xh = reinterpret_cast<int8_t*>(smem);
  uint8_t* xl = smem;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem);

  while (true) {
    // ---- next entry of this warp's sequence
    int e = 0;
    if (lane == 0) {
      if (ws.rd >= ws.wr) ws.schedule(c, widx, W, q, kLook);
      e = ws.rd >= ws.wr ? TI_UNIT_END : q[ws.rd % kCQ];
      ++ws.rd;
    }
    e = __shfl_sync(0xffffffffu, e, 0);
    if ((e == TI_UNIT_END || (e & kUnitMask) == kUnitMask) && cur_op >= 0) {
      const GemvParams& pp = c.op[cur_op];
      // this warp has sent everything it owns of the previous product: collect the all-reduce, unless the next
      // product does so itself while staging (xll)
      const bool handed = e != TI_UNIT_END && c.op[e >> 26].xll;
      if (pp.epi == EPI_ROWPAR && pp.tp > 1 && !handed) rowpar_reduce(pp, cta, ncta);
    }
    if (e == TI_UNIT_END) break;
    const int op = e >> 26, unit = e & kUnitMask;
    const GemvParams& p = c.op[op];
    if (unit == kUnitMask) {
      cur_op = op;
      tcount = 0;
      if (stamp) p0.dbg[cta * 32 + 8 + 4 * op] = globaltimer_ns();
      if (lane == 0)                              // start streaming this product's first unit while waiting
        for (int s = ws.idx - (int)cidx; s < stages; ++s) ws.next(c, widx, W, q, ring_u32, bar0, stages);
      // ---- product boundary: every warp of every CTA is done with the previous product
      if (op > 0 && p.xll) {
        // the packets of the previous product are their own synchronisation: no grid barrier.  Every CTA adds
        // them up (rank order) with the residual and writes the row(s) out; it then stages from what it wrote.
        __syncthreads();                            // the CTA's warps are done with the staged x of that product
        rowpar_reduce(c.op[op - 1], 0, 1);
        __syncthreads();
      } else if (op > 0) {
        grid_barrier(p0.sched + 2, ++nbar * ncta, p0.status, p0.dbg != nullptr && op <= 3 ? p0.dbg + cta * 32 + 1 + op : nullptr);   // stamps 2..4
      } else {
        __syncthreads();
      }
      if (stamp) p0.dbg[cta * 32 + 9 + 4 * op] = globaltimer_ns();
      lstride = limb_stride(p.K);
      xl = smem + (size_t)p.M * lstride;
      if (WT == W_INT8) stage_limbs(p, 0, p.K, xh, xl, lstride, scratch);
      else if (p.xmode == XNORM) stage_bf16_norm(p, xs, p.K + 8, scratch);
      if (WT == W_INT8) {
        inv0 = g < p.M ? scratch[288 + g] : 0.f;
        inv1 = g + 8 < p.M ? scratch[288 + g + 8] : 0.f;
      }
      if (stamp) p0.dbg[cta * 32 + 10 + 4 * op] = globaltimer_ns();
      continue;
    }
    if (lane == 0)                                // keep the ring full
      for (int s = ws.idx - (int)cidx; s < stages; ++s) ws.next(c, widx, W, q, ring_u32, bar0, stages);

    const bool hi = p.M > 8;
    const bool fine = stamp && op <= 1;           // fine-grained stamps of warp 0's last unit of products 0 and 1
    if (fine) p0.dbg[cta * 32 + 24 + 4 * op] = globaltimer_ns();
    const int grp = unit;
    int kt0, kt1;
    my_slice(tb, op, kt0, kt1);
    kt1 += kt0;
    const int rn = min(p.R, p.n_tiles - grp * p.R);
    // rows of the staged activations this lane feeds to the MMA (rows >= M are clamped: their results
    // are never written)
    const uint32_t xrow0 = (uint32_t)min(g, p.M - 1), xrow1 = (uint32_t)min(g + 8, p.M - 1);
    const uint32_t xh0 = smem_u32(xh) + xrow0 * (uint32_t)lstride + t * 16, xl0 = smem_u32(xl) + xrow0 * (uint32_t)lstride + t * 16;
    const uint32_t xh1 = smem_u32(xh) + xrow1 * (uint32_t)lstride + t * 16, xl1 = smem_u32(xl) + xrow1 * (uint32_t)lstride + t * 16;
    const uint32_t xs0 = smem_u32(xs) + (xrow0 * (uint32_t)(p.K + 8) + t * 8) * 2, xs1 = smem_u32(xs) + (xrow1 * (uint32_t)(p.K + 8) + t * 8) * 2;
    for (int r = 0; r < rn; ++r) {
      EpiPre pre{1.f, 1.f, 0u, 0u};
      if (p.T == 1 || warp % p.T == 0) pre = epi_prefetch(p, grp * p.R + r, g, t);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      int ah[2][4], al[2][4];                    // two accumulator sets: consecutive tiles do not chain
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) ah[a][b] = al[a][b] = 0;
      for (int tile0 = kt0; tile0 < kt1; tile0 += kTPS) {
        const int ntile = min(kTPS, kt1 - tile0);
        if (alive) alive = mbar_wait(bar0 + cst * 8, cpar, 2000000000ull, p.status);
        if (fine && tile0 == kt0) p0.dbg[cta * 32 + 25 + 4 * op] = globaltimer_ns();
        const uint32_t sbuf = ring_u32 + cst * (kTPS * 512u) + lane * 16;
        if (WT == W_INT8) {
          const uint32_t o = (uint32_t)tile0 * 64u;
          if (!hi) {
#pragma unroll
            for (int u = 0; u < kTPS; ++u) {
              if (u < ntile) {
                const uint4 wv = lds128(sbuf + u * 512), h0 = lds128(xh0 + o + u * 64), l0 = lds128(xl0 + o + u * 64);
                imma_s8s8(ah[u & 1], h0.x, 0u, h0.y, 0u, wv.x, wv.y);
                imma_u8s8(al[u & 1], l0.x, 0u, l0.y, 0u, wv.x, wv.y);
                imma_s8s8(ah[u & 1], h0.z, 0u, h0.w, 0u, wv.z, wv.w);
                imma_u8s8(al[u & 1], l0.z, 0u, l0.w, 0u, wv.z, wv.w);
              }
            }
          } else {
#pragma unroll
            for (int u = 0; u < kTPS; ++u) {
              if (u < ntile) {
                const uint4 wv = lds128(sbuf + u * 512), h0 = lds128(xh0 + o + u * 64), l0 = lds128(xl0 + o + u * 64);
                const uint4 h1 = lds128(xh1 + o + u * 64), l1 = lds128(xl1 + o + u * 64);
                imma_s8s8(ah[u & 1], h0.x, h1.x, h0.y, h1.y, wv.x, wv.y);
                imma_u8s8(al[u & 1], l0.x, l1.x, l0.y, l1.y, wv.x, wv.y);
                imma_s8s8(ah[u & 1], h0.z, h1.z, h0.w, h1.w, wv.z, wv.w);
                imma_u8s8(al[u & 1], l0.z, l1.z, l0.w, l1.w, wv.z, wv.w);
              }
            }
          }
        } else {
#pragma unroll
          for (int u = 0; u < kTPS; ++u) {
            if (u < ntile) {
              const uint4 wv = lds128(sbuf + u * 512);
              const int k0 = (tile0 + u) * 32;
              uint4 xv, yv = make_uint4(0, 0, 0, 0);
              if (p.xmode == XNORM) {
                xv = lds128(xs0 + k0 * 2);
                if (hi) yv = lds128(xs1 + k0 * 2);
              } else {
                xv = ld_x16(p.x + (size_t)xrow0 * p.ldx + k0 + t * 8);
                if (hi) yv = ld_x16(p.x + (size_t)xrow1 * p.ldx + k0 + t * 8);
              }
              mma_bf16_16816(acc, xv.x, yv.x, xv.y, yv.y, wv.x, wv.y);
              mma_bf16_16816(acc, xv.z, yv.z, xv.w, yv.w, wv.z, wv.w);
            }
          }
        }
        __syncwarp();                            // every lane is done with the stage before it is refilled
        ++cidx;
        if (++cst == (uint32_t)stages) {
          cst = 0;
          cpar ^= 1u;
        }
        if (lane == 0) ws.next(c, widx, W, q, ring_u32, bar0, stages);
      }
      if (fine) p0.dbg[cta * 32 + 26 + 4 * op] = globaltimer_ns();
      if (WT == W_INT8) {
#pragma unroll
        for (int b = 0; b < 4; ++b)
          acc[b] = ((float)(ah[0][b] + ah[1][b]) * 256.f + (float)(al[0][b] + al[1][b])) * (b < 2 ? inv0 : inv1);
      }
      if (p.T > 1) {
        // partial sums of the team meet in shared memory (two alternating slots: the barrier of exchange n+1
        // orders the leader's reads of slot n before anybody's writes of exchange n+2)
        // (the slot is the parity of the team's exchange count WITHIN this product: teams of different sizes in
        // consecutive products are made of warps with different histories)
        const int slot = (int)(tcount++ & 1u);
        float4* ex = tscr + (size_t)slot * kWarps * 32;
        ex[warp * 32 + lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        const int team = warp / p.T;
        asm volatile("bar.sync %0, %1;\n" ::"r"(1 + team), "r"(p.T * 32) : "memory");
        if (warp % p.T == 0) {
          for (int j = 1; j < p.T; ++j) {
            const float4 v = ex[(warp + j) * 32 + lane];
            acc[0] += v.x;
            acc[1] += v.y;
            acc[2] += v.z;
            acc[3] += v.w;
          }
          if (p.epi != EPI_ARGMAX) epilogue(p, grp * p.R + r, g, t, acc, pre);
        }
      } else if (p.epi != EPI_ARGMAX) {
        epilogue(p, grp * p.R + r, g, t, acc, pre);
      }
      if (p.epi == EPI_ARGMAX && (p.T == 1 || warp % p.T == 0)) {
        const int n = (grp * p.R + r) * 8 + 2 * t;
        if (n < p.N) {
          const float a0 = acc[0] * pre.s0, a1 = acc[1] * pre.s1, b0 = acc[2] * pre.s0, b1 = acc[3] * pre.s1;
          if (a0 > am_v0 || (a0 == am_v0 && n < am_i0)) { am_v0 = a0; am_i0 = n; }
          if (n + 1 < p.N && (a1 > am_v0 || (a1 == am_v0 && n + 1 < am_i0))) { am_v0 = a1; am_i0 = n + 1; }
          if (b0 > am_v1 || (b0 == am_v1 && n < am_i1)) { am_v1 = b0; am_i1 = n; }
          if (n + 1 < p.N && (b1 > am_v1 || (b1 == am_v1 && n + 1 < am_i1))) { am_v1 = b1; am_i1 = n + 1; }
        }
      }
    }
    if (stamp) p0.dbg[cta * 32 + 11 + 4 * op] = globaltimer_ns();
  }
  if (stamp) p0.dbg[cta * 32 + 5] = globaltimer_ns();
  // the last CTA of the launch resets the tickets and the barrier counter for the next launch
  __syncthreads();
  const GemvParams& pl = c.op[c.n_ops - 1];
  if (pl.epi == EPI_ARGMAX) {
    // (an arg-max product is the last of its launch) warp -> shared memory -> one candidate per row of this CTA
    float* sv = scratch;                                    // [kWarps][16] values, then [kWarps][16] columns
    int* si = reinterpret_cast<int*>(scratch + kWarps * 16);
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      const float ov0 = __shfl_xor_sync(0xffffffffu, am_v0, o), ov1 = __shfl_xor_sync(0xffffffffu, am_v1, o);
      const int oi0 = __shfl_xor_sync(0xffffffffu, am_i0, o), oi1 = __shfl_xor_sync(0xffffffffu, am_i1, o);
      if (ov0 > am_v0 || (ov0 == am_v0 && oi0 < am_i0)) { am_v0 = ov0; am_i0 = oi0; }
      if (ov1 > am_v1 || (ov1 == am_v1 && oi1 < am_i1)) { am_v1 = ov1; am_i1 = oi1; }
    }
    if (t == 0) {
      sv[warp * 16 + g] = am_v0;
      si[warp * 16 + g] = am_i0;
      sv[warp * 16 + g + 8] = am_v1;
      si[warp * 16 + g + 8] = am_i1;
    }
    __syncthreads();
    if (tid < pl.M) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int w = 0; w < kWarps; ++w) {
        const float v = sv[w * 16 + tid];
        const int i = si[w * 16 + tid];
        if (v > bv || (v == bv && i < bi)) {
          bv = v;
          bi = i;
        }
      }
      static_cast<float*>(pl.out)[(size_t)tid * pl.ldo + cta] = bv;
      pl.out_idx[(size_t)tid * pl.ldo + cta] = bi == 0x7fffffff ? -1 : bi;
    }
  }
  if (tid == 0) {
    __threadfence();
    const int fin = atomicAdd(p0.sched + 1, 1);
    if ((fin + 1) % ncta == 0) {
      for (int i = 0; i < kMaxChain * 16; ++i) p0.sched[8 + i] = 0;
      p0.sched[2] = 0;
      __threadfence();
    }
  }
}

template <int WT>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(const __grid_constant__ ChainParams c) {
  extern __shared__ __align__(128) uint8_t smem[];
  gemv_body<WT>(c, blockIdx.x, gridDim.x, smem);
}

// All emulated ranks of a tensor-parallel group in ONE cooperative launch on one GPU: block b
// works for rank b / ctas_per_rank.  Used by tests where fewer GPUs than ranks are available;
// separate launches that wait on one another must never share a GPU.
template <int WT>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel_ranks(const ChainParams* clist, int ctas_per_rank) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int r = blockIdx.x / ctas_per_rank;
  gemv_body<WT>(clist[r], blockIdx.x - r * ctas_per_rank, ctas_per_rank, smem);
}

static int op_x_bytes(const GemvParams& p, int wt) { return (int)x_smem_bytes_impl(wt, p.xmode, p.M, p.K, p.K); }

static size_t smem_bytes(const ChainParams& c) {
  const GemvParams& p = c.op[0];
  bool team = false;
  for (int i = 0; i < c.n_ops; ++i) team = team || c.op[i].T > 1;
  return (size_t)c.x_bytes + (size_t)kWarps * (p.stages * (p.tps * 512 + 8) + kCQ * 4) + (team ? kTeamBytes : 0);
}

static int check(const GemvParams& p, int wt) {
  const int tk = wt == W_INT8 ? 64 : 32;
  if (p.M < 1 || p.M > 16 || p.N < 2 || (p.N & 1) || p.K % tk || p.KB * tk != p.K) return -2;
  if (p.R < 1 || p.R > kMaxR || p.n_tiles < 1 || p.n_tiles >= (1 << 26)) return -3;
  if (p.S != 1 || p.kb_per_split != p.KB) return -6;
  if (p.T < 1 || p.T > kWarps || p.KB < p.T) return -6;
  if ((p.n_tiles + p.R - 1) / p.R >= kUnitMask) return -3;
  if (p.tps != kTPS) return -7;
  if (p.sched == nullptr || p.stages < 1 || p.stages > kMaxStages) return -7;
  if (p.xmode < 0 || p.xmode > 1 || p.epi < 0 || p.epi > 4) return -8;
  if (p.epi == EPI_ARGMAX && p.out_idx == nullptr) return -8;
  if (p.K % 8 || p.ldx % 8) return -4;
  if (p.tp > kMaxRanks || (p.tp > 1 && p.M > p.m_cap)) return -5;
  return 0;
}

static int prepare(ChainParams& c, int wt) {
  if (c.n_ops < 1 || c.n_ops > kMaxChain) return -9;
  int xb = 0;
  for (int i = 0; i < c.n_ops; ++i) {
    const int rc = check(c.op[i], wt);
    if (rc) return rc;
    if (c.op[i].sched != c.op[0].sched || c.op[i].stages != c.op[0].stages || c.op[i].tps != c.op[0].tps) return -9;
    if (c.op[i].xll) {
      if (i == 0) return -10;
      const GemvParams &q = c.op[i - 1], &p = c.op[i];
      if (q.epi != EPI_ROWPAR || q.tp < 2 || q.M != p.M || q.N != p.K || q.out != (void*)p.x || p.ldx != q.N) return -10;
    }
    if (c.op[i].epi == EPI_ARGMAX && i != c.n_ops - 1) return -11;     // an arg-max product closes its launch
    xb = std::max(xb, op_x_bytes(c.op[i], wt));
  }
  c.x_bytes = xb;
  if (smem_bytes(c) > 227 * 1024 - 4096) return -4;      // 4 KB are static (queues' tables, reduction scratch)
  return 0;
}

template <int WT>
static int launch(const ChainParams& c, int ncta, cudaStream_t st, const ChainParams* dev_list, int nranks) {
  const size_t sm = smem_bytes(c);
  static bool configured = false, configured_ranks = false;
  if (dev_list == nullptr) {
    auto k = gemv_kernel<WT>;
    if (!configured) {
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 4096);
      configured = true;
    }
    cudaError_t e = launch_kernel(k, dim3(ncta), dim3(kThreads), sm, st, true, c);
    if (e != cudaSuccess) return (int)e;
  } else {
    auto k = gemv_kernel_ranks<WT>;
    if (!configured_ranks) {
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 4096);
      configured_ranks = true;
    }
    void* args[] = {(void*)&dev_list, (void*)&ncta};
    cudaError_t e = cudaLaunchCooperativeKernel((void*)k, dim3(ncta * nranks), dim3(kThreads), args, sm, st);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cudaGetLastError();
}

}  // namespace ti

extern "C" {

int ti_gemv_params_size() { return (int)sizeof(ti::GemvParams); }
int ti_chain_params_size() { return (int)sizeof(ti::ChainParams); }

// Runs c->n_ops dependent products (y_i = x_i W_i^T with their prologues / epilogues) in one launch.
// `c` is modified (x_bytes is filled in).  Returns 0 or a CUDA / argument error code.
int ti_gemv_chain(ti::ChainParams* c, int wt, int ncta, void* stream) {
  const int rc = ti::prepare(*c, wt);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return wt == ti::W_INT8 ? ti::launch<ti::W_INT8>(*c, ncta, st, nullptr, 1) : ti::launch<ti::W_BF16>(*c, ncta, st, nullptr, 1);
}

// Size `c` exactly as ti_gemv_chain would (validation + x_bytes) without launching.
int ti_gemv_chain_prepare(ti::ChainParams* c, int wt, int ncta) { return ti::prepare(*c, wt); }

// One cooperative launch that runs `nranks` emulated ranks (prepared chain blocks in device memory at
// `dev_chains`, a host copy of rank 0's block in `c0`) with `ncta` blocks each.  int8 weights only.
int ti_gemv_ranks(ti::ChainParams* c0, const ti::ChainParams* dev_chains, int nranks, int ncta, void* stream) {
  const int rc = ti::prepare(*c0, ti::W_INT8);
  if (rc) return rc;
  return ti::launch<ti::W_INT8>(*c0, ncta, static_cast<cudaStream_t>(stream), dev_chains, nranks);
}

}  // extern "C"
