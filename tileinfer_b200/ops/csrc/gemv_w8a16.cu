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
  int J;                         // k-slices a CTA group owns (S % J == 0): CTA c stages slice c % J of x
  unsigned long long* dbg;       // optional [ncta][8] globaltimer stamps of warp 0 (profiling aid)
  int* sched;                    // dynamic scheduling state: [0] launches finished, [1] CTAs finished, [8 + 3*16] tickets
  int tps;                       // 512-byte tiles per ring stage (4, 8 or 16)
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
enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_ROWPAR = 2, EPI_F32 = 3 };
enum { W_INT8 = 0, W_BF16 = 1 };

constexpr int kThreads = 256;
constexpr int kMaxTilesPerStage = 16;
constexpr int kQueue = 16;                 // per-warp queue of fetched unit indices

template <int EPI>
TI_DEVICE void epilogue(const GemvParams& p, int nt, int g, int t, const float (&acc)[4]) {
  const int n = nt * 8 + 2 * t;
  if (n >= p.N) return;
  float s0 = 1.f, s1 = 1.f;
  if (p.scale != nullptr) {
    s0 = bf16_to_f(p.scale[n]);
    s1 = bf16_to_f(p.scale[n + 1]);
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = g + half * 8;
    if (m >= p.M) continue;
    float v0 = acc[half * 2] * s0, v1 = acc[half * 2 + 1] * s1;
    if (EPI == EPI_STORE) {
      uint32_t* o = reinterpret_cast<uint32_t*>(static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldo + n);
      *o = pack_bf16(v0, v1);
    } else if (EPI == EPI_F32) {
      float2* o = reinterpret_cast<float2*>(static_cast<float*>(p.out) + (size_t)m * p.ldo + n);
      *o = make_float2(v0, v1);
    } else if (EPI == EPI_SWIGLU) {
      // rows come interleaved (gate, up); both are rounded to bf16 first, as a separate activation
      // kernel reading bf16 projections would see them
      const float gate = round_bf16(v0), up = round_bf16(v1);
      static_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + (n >> 1)] = __float2bfloat16_rn(silu_f(gate) * up);
    } else {  // EPI_ROWPAR
      float sum0 = v0, sum1 = v1;
      if (p.tp > 1) {
        const unsigned tag = (*p.step_ptr) * 65536u + (unsigned)p.order + 1u;
        const int slot = p.order & 1;
        const size_t pairs = (size_t)(p.N >> 1);
        const size_t mine = (((size_t)slot * p.tp + p.rank) * p.m_cap + m) * pairs + (n >> 1);
        for (int q = 0; q < p.tp; ++q)
          if (q != p.rank) ll_store2(reinterpret_cast<uint8_t*>(p.peer_ll[q]) + mine * 16, v0, v1, tag);
        sum0 = 0.f;
        sum1 = 0.f;
        const uint8_t* local = reinterpret_cast<const uint8_t*>(p.peer_ll[p.rank]);
        for (int r = 0; r < p.tp; ++r) {   // fixed rank order: every rank gets the same bits
          float a = v0, b = v1;
          if (r != p.rank) {
            const size_t idx = (((size_t)slot * p.tp + r) * p.m_cap + m) * pairs + (n >> 1);
            ll_wait2(local + idx * 16, tag, a, b, p.timeout_ns, p.status);
          }
          sum0 += a;
          sum1 += b;
        }
      }
      const uint32_t rw = *reinterpret_cast<const uint32_t*>(p.resid + (size_t)m * p.N + n);
      uint32_t* o = reinterpret_cast<uint32_t*>(static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.N + n);
      *o = pack_bf16(bf16lo(rw) + sum0, bf16hi(rw) + sum1);
    }
  }
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

// ---------------------------------------------------------------- work decomposition
// A unit is (row tile nt, k-split ks).  CTAs form J groups (group j = CTAs with cta % J == j); group j
// owns the k-splits [j*S/J, (j+1)*S/J) and stages only that slice of x.  Inside a group the units are
// dealt round-robin to the warps.
struct Group {
  int j, ssub, widx, wcount, units, kbs0, kbs1;
};
TI_DEVICE Group make_group(const GemvParams& p, int cta, int ncta, int warp, int nwarps) {
  Group gr;
  gr.j = cta % p.J;
  gr.ssub = p.S / p.J;
  gr.widx = (cta / p.J) * nwarps + warp;
  gr.wcount = ((ncta - gr.j + p.J - 1) / p.J) * nwarps;
  gr.units = p.n_tiles * gr.ssub;
  gr.kbs0 = min(p.KB, gr.j * gr.ssub * p.kb_per_split);
  gr.kbs1 = min(p.KB, gr.kbs0 + gr.ssub * p.kb_per_split);
  return gr;
}
struct Unit { int nt, ks, kb0, nkb; };
TI_DEVICE Unit unit_of(const GemvParams& p, const Group& gr, int ul) {
  Unit u;
  u.nt = ul / gr.ssub;
  u.ks = gr.j * gr.ssub + (ul - u.nt * gr.ssub);
  u.kb0 = u.ks * p.kb_per_split;
  u.nkb = max(0, min(p.KB, u.kb0 + p.kb_per_split) - u.kb0);
  return u;
}

// Cursor of the warp-private weight stream (used by lane 0 only).  Units are handed out dynamically:
// a ticket counter per CTA group is advanced with atomicAdd, so a warp that falls behind (slow HBM
// channel, long epilogue wait) simply takes fewer units.  Fetched unit indices go through a small
// queue so that the consuming side sees them in the same order; each unit is cut into chunks of at
// most `tps` consecutive 512-byte tiles that the TMA engine copies into the ring, stage after stage.
struct IssueCursor {
  int ul, tile, nkb, idx, wr, rd, pre;
  bool done, can_fetch;
  size_t base;
  // The first unit of every warp is assigned statically (unit = warp index in its group), so its
  // weights can be requested before the kernel is allowed to look at any mutable state; tickets then
  // number the remaining units from gr.wcount on.
  TI_DEVICE void take_static(const GemvParams& p, const Group& gr, volatile int* q) {
    ul = -1;
    if (gr.widx >= gr.units) return;
    q[wr++ % kQueue] = gr.widx;
    const Unit un = unit_of(p, gr, gr.widx);
    if (un.nkb > 0) {
      ul = gr.widx;
      nkb = un.nkb;
      base = ((size_t)un.nt * p.KB + un.kb0) * 512;
      tile = 0;
    }
  }
  TI_DEVICE void fetch(const GemvParams& p, const Group& gr, int* ticket, volatile int* q) {
    ul = -1;
    while (!done && wr - rd < kQueue - 1) {
      const int u = gr.wcount + pre;     // ticket drawn one unit ago: its latency is already paid
      pre = atomicAdd(ticket, 1);
      if (u >= gr.units) {
        q[wr++ % kQueue] = -1;
        done = true;
        return;
      }
      q[wr++ % kQueue] = u;
      const Unit un = unit_of(p, gr, u);
      if (un.nkb > 0) {
        ul = u;
        nkb = un.nkb;
        base = ((size_t)un.nt * p.KB + un.kb0) * 512;
        tile = 0;
        return;
      }
    }
  }
  TI_DEVICE void next(const GemvParams& p, const Group& gr, int* ticket, volatile int* q, uint32_t ring_u32,
                      uint32_t bar0, int stages) {
    if (ul < 0 && can_fetch) fetch(p, gr, ticket, q);
    if (ul < 0) return;
    const int ntile = min(p.tps, nkb - tile);
    const uint32_t st = (uint32_t)idx % (uint32_t)stages;
    const uint32_t bytes = (uint32_t)ntile * 512u;
    mbar_expect_tx(bar0 + st * 8, bytes);
    bulk_g2s(ring_u32 + st * (uint32_t)p.tps * 512u, p.w + base + (size_t)tile * 512, bytes, bar0 + st * 8);
    ++idx;
    tile += ntile;
    if (tile >= nkb) ul = -1;
  }
};

// ---------------------------------------------------------------- activation staging
// Per-row statistics scratch: red[nwarps][16] then rowv[16] (rrms), rows[16] (limb scale 2^(e-14)).
template <int XMODE>
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
template <int XMODE>
TI_DEVICE void stage_limbs(const GemvParams& p, int k_lo, int k_hi, int8_t* xh, uint8_t* xl, int stride, float* scratch) {
  const int tid = threadIdx.x;
  float* red = scratch;            // [16 warps][16]
  float* rrms = scratch + 256;     // [16]
  float* amax = scratch + 272;     // [16]
  float* inv = scratch + 288;      // [16]  2^(e-14): value of one fixed-point unit
  const int nthreads = blockDim.x;
  // ---- single-row fast path (batch-1 decode): the row lives in registers, read from memory once
  if (p.M == 1 && (k_hi - k_lo) <= 40 * nthreads && (XMODE != XNORM || (k_lo == 0 && k_hi == p.K))) {
    const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
    const int c_lo = k_lo >> 3, c_hi = k_hi >> 3;
    float v[5][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 5; ++j) {
      const int c = c_lo + tid + j * nthreads;
      uint4 q = make_uint4(0, 0, 0, 0);
      if (c < c_hi) q = ldg_cached16(p.x + (size_t)c * 8);
      const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[j][2 * i] = bf16lo(w4[i]);
        v[j][2 * i + 1] = bf16hi(w4[i]);
        ss += v[j][2 * i] * v[j][2 * i] + v[j][2 * i + 1] * v[j][2 * i + 1];
      }
    }
    if (XMODE == XNORM) {
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
        const uint4 nw = ldg_cached16(p.norm_w + (size_t)c * 8);
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
  if (XMODE == XNORM) {
#pragma unroll
    for (int m = 0; m < 16; ++m) acc[m] = 0.f;
    for (int c = tid; c < (p.K >> 3); c += blockDim.x) {
#pragma unroll
      for (int m = 0; m < 16; ++m) {
        if (m >= p.M) break;
        const uint4 v = ldg_cached16(p.x + (size_t)m * p.ldx + c * 8);
        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m] += bf16lo(w4[i]) * bf16lo(w4[i]) + bf16hi(w4[i]) * bf16hi(w4[i]);
      }
    }
    block_row_reduce<XMODE>(acc, p.M, red, rrms, tid, false);
    if (tid < p.M) rrms[tid] = rsqrtf(rrms[tid] / (float)p.K + p.eps);
    __syncthreads();
  }
  // pass A: row maxima over the slice
#pragma unroll
  for (int m = 0; m < 16; ++m) acc[m] = 0.f;
  const int c_lo = k_lo >> 3, c_hi = k_hi >> 3;
  for (int c = c_lo + tid; c < c_hi; c += blockDim.x) {
    uint4 nw = make_uint4(0, 0, 0, 0);
    if (XMODE == XNORM) nw = ldg_cached16(p.norm_w + c * 8);
    const uint32_t n4[4] = {nw.x, nw.y, nw.z, nw.w};
#pragma unroll
    for (int m = 0; m < 16; ++m) {
      if (m >= p.M) break;
      const uint4 v = ldg_cached16(p.x + (size_t)m * p.ldx + c * 8);
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
      const float rr = XMODE == XNORM ? rrms[m] : 1.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float a = bf16lo(w4[i]), b = bf16hi(w4[i]);
        if (XMODE == XNORM) {
          a = round_bf16(a * rr * (1.f + bf16lo(n4[i])));
          b = round_bf16(b * rr * (1.f + bf16hi(n4[i])));
        }
        acc[m] = fmaxf(acc[m], fmaxf(fabsf(a), fabsf(b)));
      }
    }
  }
  block_row_reduce<XMODE>(acc, p.M, red, amax, tid, true);
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
    if (XMODE == XNORM) nw = ldg_cached16(p.norm_w + c * 8);
    const uint32_t n4[4] = {nw.x, nw.y, nw.z, nw.w};
#pragma unroll
    for (int m = 0; m < 16; ++m) {
      if (m >= p.M) break;
      const uint4 v = ldg_cached16(p.x + (size_t)m * p.ldx + c * 8);
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
      const float rr = XMODE == XNORM ? rrms[m] : 1.f, qs = amax[m];
      uint32_t hw[2] = {0, 0}, lw[2] = {0, 0};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float a = bf16lo(w4[i]), b = bf16hi(w4[i]);
        if (XMODE == XNORM) {
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
      const uint4 v = ldg_cached16(p.x + (size_t)m * p.ldx + c * 8);
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m] += bf16lo(w4[i]) * bf16lo(w4[i]) + bf16hi(w4[i]) * bf16hi(w4[i]);
    }
  }
  block_row_reduce<XNORM>(acc, p.M, red, rrms, tid, false);
  if (tid < p.M) rrms[tid] = rsqrtf(rrms[tid] / (float)p.K + p.eps);
  __syncthreads();
  for (int c = tid; c < chunks; c += blockDim.x) {
    const uint4 nw = ldg_cached16(p.norm_w + c * 8);
    const uint32_t n4[4] = {nw.x, nw.y, nw.z, nw.w};
    for (int m = 0; m < rows; ++m) {
      uint4 o = make_uint4(0, 0, 0, 0);
      if (m < p.M) {
        const uint4 v = ldg_cached16(p.x + (size_t)m * p.ldx + c * 8);
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

// ---------------------------------------------------------------- split-k bookkeeping
// The warp that brings a row tile's arrival counter to S sums the S partials in a fixed order
// (deterministic) and runs the epilogue.
TI_DEVICE int splitk_announce(const GemvParams& p, int pend_nt, unsigned& tk_val, int lane) {
  if (pend_nt < 0) return -1;
  __threadfence();
  __syncwarp();
  if (lane == 0) tk_val = atomicAdd(p.counters + pend_nt, 1u);
  return pend_nt;
}
template <int EPI>
TI_DEVICE void splitk_settle(const GemvParams& p, int tk_nt, unsigned tk_val, int g, int t, int lane) {
  if (tk_nt < 0) return;
  const unsigned prev = __shfl_sync(0xffffffffu, tk_val, 0);
  if (prev != (unsigned)p.S - 1u) return;
  __threadfence();
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < p.S; ++s) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(p.ws + ((size_t)tk_nt * p.S + s) * 128 + lane * 4));
    sum[0] += v.x; sum[1] += v.y; sum[2] += v.z; sum[3] += v.w;
  }
  if (lane == 0) p.counters[tk_nt] = 0u;
  epilogue<EPI>(p, tk_nt, g, t, sum);
}

// ---------------------------------------------------------------- main body
template <int WT, int XMODE, int EPI>
TI_DEVICE void gemv_body(const GemvParams& p, int cta, int ncta, uint8_t* smem) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int nwarps = blockDim.x >> 5;
  const bool hi = p.M > 8;
  const Group gr = make_group(p, cta, ncta, warp, nwarps);
  const bool stamp = p.dbg != nullptr && tid == 0;
  if (stamp) p.dbg[cta * 8 + 0] = globaltimer_ns();
  const int kslice = (gr.kbs1 - gr.kbs0) * (WT == W_INT8 ? 64 : 32);
  const int kslice_max = min(p.KB, (p.S / p.J) * p.kb_per_split) * (WT == W_INT8 ? 64 : 32);
  const size_t x_bytes = x_smem_bytes_impl(WT, XMODE, p.M, p.K, kslice_max);

  // ---- weight stream first: the ring fills while the activations are being staged
  const int stages = p.stages;
  const int stage_bytes = p.tps * 512;
  uint8_t* ring = smem + x_bytes + (size_t)warp * stages * stage_bytes;
  const uint32_t ring_u32 = smem_u32(ring);
  uint8_t* after_ring = smem + x_bytes + (size_t)nwarps * stages * stage_bytes;
  const uint32_t bar0 = smem_u32(after_ring) + warp * stages * 8;
  volatile int* queue = reinterpret_cast<volatile int*>(after_ring + nwarps * stages * 8) + warp * kQueue;
  IssueCursor issue;
  issue.ul = -1;
  issue.idx = issue.wr = issue.rd = 0;
  issue.nkb = issue.tile = 0;
  issue.base = 0;
  issue.done = false;
  issue.can_fetch = false;
  issue.pre = 0;
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(bar0 + s * 8, 1);
    fence_mbar_init();
    issue.take_static(p, gr, queue);
    for (int s = 0; s < stages; ++s) issue.next(p, gr, nullptr, queue, ring_u32, bar0, stages);
  }
  __syncwarp();
  // Everything above touched only weights and this CTA's shared memory.  Let the next kernel of the
  // stream start its own prefetch, then wait until the previous kernel (which produced x and may still
  // be using the split-k workspace, the arrival counters and the tickets) has completed.
  pdl_trigger();
  pdl_wait();
  if (stamp) p.dbg[cta * 8 + 1] = globaltimer_ns();
  // ticket counters rotate over three slots: this launch uses slot (launches finished) % 3, which the
  // previous launch zeroed, and zeroes the slot of the next launch
  const int seq = *reinterpret_cast<volatile int*>(p.sched);
  int* ticket = p.sched + 8 + (seq % 3) * 16 + gr.j;
  if (cta == 0 && tid < 16) p.sched[8 + ((seq + 1) % 3) * 16 + tid] = 0;
  if (lane == 0) {
    issue.pre = atomicAdd(ticket, 1);
    issue.can_fetch = true;
  }

  // ---- activations
  float* scratch = reinterpret_cast<float*>(smem + x_bytes - 2048);
  const int lstride = limb_stride(kslice_max);
  int8_t* xh = reinterpret_cast<int8_t*>(smem);
  uint8_t* xl = smem + (size_t)p.M * lstride;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem);
  const int xs_stride = p.K + 8;
  if (WT == W_INT8) {
    stage_limbs<XMODE>(p, gr.kbs0 * 64, gr.kbs0 * 64 + kslice, xh, xl, lstride, scratch);
  } else if (XMODE == XNORM) {
    stage_bf16_norm(p, xs, xs_stride, scratch);
  }
  float inv0 = 0.f, inv1 = 0.f;                 // value of one fixed-point unit for rows g and g+8
  if (WT == W_INT8) {
    inv0 = g < p.M ? scratch[288 + g] : 0.f;
    inv1 = g + 8 < p.M ? scratch[288 + g + 8] : 0.f;
  }

  if (stamp) p.dbg[cta * 8 + 2] = globaltimer_ns();
  if (lane == 0)                                // top the ring up if the static unit was a short one
    for (int s = issue.idx; s < stages; ++s) issue.next(p, gr, ticket, queue, ring_u32, bar0, stages);
  unsigned cidx = 0;                            // chunks consumed by this warp so far
  bool alive = true;
  int pend_nt = -1, tk_nt = -1;                 // split-k: partial written / arrival in flight
  unsigned tk_val = 0;
  while (true) {
    int ul = 0;
    if (lane == 0) {
      if (issue.rd == issue.wr) issue.fetch(p, gr, ticket, queue);   // queue drained by empty units
      ul = queue[issue.rd++ % kQueue];
    }
    ul = __shfl_sync(0xffffffffu, ul, 0);
    if (ul < 0) break;
    const Unit un = unit_of(p, gr, ul);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int ah[4] = {0, 0, 0, 0}, al[4] = {0, 0, 0, 0};
    for (int tile0 = 0; tile0 < un.nkb; tile0 += p.tps) {
      const int ntile = min(p.tps, un.nkb - tile0);
      const unsigned st = cidx % (unsigned)stages;
      if (alive) alive = mbar_wait(bar0 + st * 8, (cidx / (unsigned)stages) & 1u, 2000000000ull, p.status);
      if (stamp && cidx == 0) p.dbg[cta * 8 + 3] = globaltimer_ns();
      const uint8_t* sbuf = ring + (size_t)st * stage_bytes + lane * 16;
#pragma unroll 4
      for (int u = 0; u < kMaxTilesPerStage; ++u) {
        if (u >= ntile) break;
        const uint4 wv = *reinterpret_cast<const uint4*>(sbuf + u * 512);
        const int kb = un.kb0 + tile0 + u;
        if (WT == W_INT8) {
          const size_t xo = (size_t)(kb - gr.kbs0) * 64 + t * 16;
          const uint4 z = make_uint4(0, 0, 0, 0);
          const uint4 h0 = g < p.M ? *reinterpret_cast<const uint4*>(xh + (size_t)g * lstride + xo) : z;
          const uint4 l0 = g < p.M ? *reinterpret_cast<const uint4*>(xl + (size_t)g * lstride + xo) : z;
          const uint4 h1 = (hi && g + 8 < p.M) ? *reinterpret_cast<const uint4*>(xh + (size_t)(g + 8) * lstride + xo) : z;
          const uint4 l1 = (hi && g + 8 < p.M) ? *reinterpret_cast<const uint4*>(xl + (size_t)(g + 8) * lstride + xo) : z;
          imma_s8s8(ah, h0.x, h1.x, h0.y, h1.y, wv.x, wv.y);
          imma_s8s8(ah, h0.z, h1.z, h0.w, h1.w, wv.z, wv.w);
          imma_u8s8(al, l0.x, l1.x, l0.y, l1.y, wv.x, wv.y);
          imma_u8s8(al, l0.z, l1.z, l0.w, l1.w, wv.z, wv.w);
        } else {
          const int k0 = kb * 32 + t * 8;
          uint4 xv, yv;
          if (XMODE == XNORM) {
            xv = *reinterpret_cast<const uint4*>(xs + (size_t)g * xs_stride + k0);
            yv = hi ? *reinterpret_cast<const uint4*>(xs + (size_t)(g + 8) * xs_stride + k0) : make_uint4(0, 0, 0, 0);
          } else {
            xv = (g < p.M) ? ldg_cached16(p.x + (size_t)g * p.ldx + k0) : make_uint4(0, 0, 0, 0);
            yv = (g + 8 < p.M) ? ldg_cached16(p.x + (size_t)(g + 8) * p.ldx + k0) : make_uint4(0, 0, 0, 0);
          }
          mma_bf16_16816(acc, xv.x, yv.x, xv.y, yv.y, wv.x, wv.y);
          mma_bf16_16816(acc, xv.z, yv.z, xv.w, yv.w, wv.z, wv.w);
        }
      }
      __syncwarp();                              // every lane is done with the stage before it is refilled
      ++cidx;
      if (lane == 0) issue.next(p, gr, ticket, queue, ring_u32, bar0, stages);
    }
    if (WT == W_INT8) {
      acc[0] = ((float)ah[0] * 256.f + (float)al[0]) * inv0;
      acc[1] = ((float)ah[1] * 256.f + (float)al[1]) * inv0;
      acc[2] = ((float)ah[2] * 256.f + (float)al[2]) * inv1;
      acc[3] = ((float)ah[3] * 256.f + (float)al[3]) * inv1;
    }
    if (p.S == 1) {
      epilogue<EPI>(p, un.nt, g, t, acc);
    } else {
      // split-k: arrivals are deferred so that neither the fence nor the counter round trip stalls the
      // stream: (a) settle the arrival issued one unit ago, (b) announce the partial written one unit
      // ago (its store has long landed, the fence is cheap), (c) write this unit's partial
      splitk_settle<EPI>(p, tk_nt, tk_val, g, t, lane);
      tk_nt = splitk_announce(p, pend_nt, tk_val, lane);
      *reinterpret_cast<float4*>(p.ws + ((size_t)un.nt * p.S + un.ks) * 128 + lane * 4) =
          make_float4(acc[0], acc[1], acc[2], acc[3]);
      pend_nt = un.nt;
    }
    if (stamp) p.dbg[cta * 8 + 4] = globaltimer_ns();
  }
  if (p.S > 1) {                                 // drain the deferred arrivals
    splitk_settle<EPI>(p, tk_nt, tk_val, g, t, lane);
    tk_nt = splitk_announce(p, pend_nt, tk_val, lane);
    splitk_settle<EPI>(p, tk_nt, tk_val, g, t, lane);
  }
  if (stamp) p.dbg[cta * 8 + 5] = globaltimer_ns();
  // the last CTA to finish advances the launch sequence number (monotonic, never reset)
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int fin = atomicAdd(p.sched + 1, 1);
    if ((fin + 1) % ncta == 0) atomicAdd(p.sched, 1);
  }
}

template <int WT, int XMODE, int EPI>
__global__ void __launch_bounds__(kThreads, 2) gemv_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  gemv_body<WT, XMODE, EPI>(p, blockIdx.x, gridDim.x, smem);
}

// All emulated ranks of a tensor-parallel group in ONE cooperative launch on one GPU: block b
// works for rank b / ctas_per_rank.  Used by tests where fewer GPUs than ranks are available;
// separate launches that wait on one another must never share a GPU.
template <int WT, int XMODE, int EPI>
__global__ void __launch_bounds__(kThreads, 2) gemv_kernel_ranks(const GemvParams* plist, int ctas_per_rank) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int r = blockIdx.x / ctas_per_rank;
  gemv_body<WT, XMODE, EPI>(plist[r], blockIdx.x - r * ctas_per_rank, ctas_per_rank, smem);
}

static size_t smem_bytes(const GemvParams& p, int wt, int xmode) {
  const int tk = wt == W_INT8 ? 64 : 32;
  const int kslice = std::min(p.KB, (p.S / p.J) * p.kb_per_split) * tk;
  return x_smem_bytes_impl(wt, xmode, p.M, p.K, kslice) + (size_t)(kThreads / 32) * (p.stages * (p.tps * 512 + 8) + kQueue * 4);
}

template <int WT, int XMODE, int EPI>
static int launch(const GemvParams& p, int ncta, cudaStream_t st, const GemvParams* dev_list, int nranks) {
  const size_t sm = smem_bytes(p, WT, XMODE);
  if (dev_list == nullptr) {
    auto k = gemv_kernel<WT, XMODE, EPI>;
    static size_t configured = 0;
    if (sm > configured) {
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      configured = 227 * 1024;
    }
    cudaError_t e = launch_kernel(k, dim3(ncta), dim3(kThreads), sm, st, true, p);
    if (e != cudaSuccess) return (int)e;
  } else {
    auto k = gemv_kernel_ranks<WT, XMODE, EPI>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    void* args[] = {(void*)&dev_list, (void*)&ncta};
    cudaError_t e = cudaLaunchCooperativeKernel((void*)k, dim3(ncta * nranks), dim3(kThreads), args, sm, st);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cudaGetLastError();
}

template <int WT, int XMODE>
static int dispatch_epi(const GemvParams& p, int epi, int ncta, cudaStream_t st, const GemvParams* dl, int nr) {
  switch (epi) {
    case EPI_STORE: return launch<WT, XMODE, EPI_STORE>(p, ncta, st, dl, nr);
    case EPI_SWIGLU: return launch<WT, XMODE, EPI_SWIGLU>(p, ncta, st, dl, nr);
    case EPI_ROWPAR: return launch<WT, XMODE, EPI_ROWPAR>(p, ncta, st, dl, nr);
    case EPI_F32: return launch<WT, XMODE, EPI_F32>(p, ncta, st, dl, nr);
  }
  return -1;
}

static int check(const GemvParams& p, int wt, int xmode, int ncta) {
  const int tk = wt == W_INT8 ? 64 : 32;
  if (p.M < 1 || p.M > 16 || p.N < 2 || (p.N & 1) || p.K % tk || p.KB * tk != p.K) return -2;
  if (p.S < 1 || p.kb_per_split < 1 || (long long)p.S * p.kb_per_split < p.KB) return -3;
  if (p.J < 1 || p.S % p.J || p.J > ncta || (wt != W_INT8 && p.J != 1)) return -6;
  if (p.tps != 4 && p.tps != 8 && p.tps != 16) return -7;
  if (p.sched == nullptr || p.J > 16) return -7;
  if (p.stages < 1 || p.stages > 8 || smem_bytes(p, wt, xmode) > 227 * 1024) return -4;
  if (p.K % 8 || p.ldx % 8) return -4;
  if (p.tp > kMaxRanks || (p.tp > 1 && p.M > p.m_cap)) return -5;
  return 0;
}

}  // namespace ti

extern "C" {

// Launches y = x W^T with the selected weight type, x source and epilogue on `stream`.
// Returns 0 or a CUDA / argument error code.
int ti_gemv(const ti::GemvParams* p, int wt, int xmode, int epi, int ncta, void* stream) {
  int rc = ti::check(*p, wt, xmode, ncta);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (wt == ti::W_INT8)
    return xmode == ti::XNORM ? ti::dispatch_epi<ti::W_INT8, ti::XNORM>(*p, epi, ncta, st, nullptr, 1)
                              : ti::dispatch_epi<ti::W_INT8, ti::XGLOBAL>(*p, epi, ncta, st, nullptr, 1);
  return xmode == ti::XNORM ? ti::dispatch_epi<ti::W_BF16, ti::XNORM>(*p, epi, ncta, st, nullptr, 1)
                            : ti::dispatch_epi<ti::W_BF16, ti::XGLOBAL>(*p, epi, ncta, st, nullptr, 1);
}

// One cooperative launch that runs `nranks` emulated ranks (parameter blocks in device memory at
// `dev_params`, a host copy of rank 0's block in `p0` for validation) with `ncta` blocks each.
int ti_gemv_ranks(const ti::GemvParams* p0, const ti::GemvParams* dev_params, int nranks, int wt, int xmode, int epi,
                  int ncta, void* stream) {
  int rc = ti::check(*p0, wt, xmode, ncta);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (wt != ti::W_INT8) return -6;
  return xmode == ti::XNORM ? ti::dispatch_epi<ti::W_INT8, ti::XNORM>(*p0, epi, ncta, st, dev_params, nranks)
                            : ti::dispatch_epi<ti::W_INT8, ti::XGLOBAL>(*p0, epi, ncta, st, dev_params, nranks);
}

int ti_gemv_params_size() { return (int)sizeof(ti::GemvParams); }

}  // extern "C"
