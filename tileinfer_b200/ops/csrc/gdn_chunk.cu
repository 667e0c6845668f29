// Chunk-parallel gated delta rule for prefill (WY / UT form), on the tensor cores.
//
// Replaces the reference's chunk kernel (kernels/gated_delta_rule_prefill.py:28-120: chunk 32, scalar FMA loops,
// and without the (v - S^T k) correction, i.e. not the delta rule) and the external flash_qla dependency
// (model/qwen_36.py:73-76).  The token-serial recurrence of gdn.cu stays for decode steps and short chunks.
//
// For a chunk of C = 64 tokens of one v-head (g = cumulative log decay inside the chunk, b = beta):
//     L[i][j]  = b_i (k_i . k_j) exp(g_i - g_j)             (i > j)
//     X        = (I + L)^-1                                   (unit lower triangular)
//     u        = X (b v)            w = X (b k exp(g))
//     v_new    = u - w S                                      S: state [dk, dv] before the chunk
//     out      = (q exp(g)) S + ((q k^T) * exp(g_i - g_j), i >= j) v_new
//     S       <- exp(g_C) S + (k exp(g_C - g))^T v_new
// Everything up to u and w does not depend on S: `gdn_chunk_prepare_kernel` computes it for ALL chunks and heads
// in parallel (causal conv + SiLU, q/k norms, gates, the two 64 x 64 Gram products, the blocked triangular inverse,
// u and w), and writes every operand of the scan in the register-fragment order of mma.sync.m16n8k16, so the scan
// fetches a fragment with one coalesced 16-byte load per lane and needs no shared-memory staging or ldmatrix.
// `gdn_chunk_scan_kernel` then walks the chunks of a sequence: one CTA per (v-head, 32 state columns, sequence),
// state slice S^T[32, dk] in fp32 accumulator registers; because the slice is kept TRANSPOSED, the accumulator
// fragment of the update is exactly the B fragment the next chunk's products need (bf16 copy in shared memory).
// `gdn_chunk_finish_kernel` applies the gated RMSNorm * silu(z); `gdn_conv_tail_kernel` writes the conv history.
// Chunks end at the block-aligned positions where a state snapshot is wanted (prefix cache), so snapshots are
// plain copies of the running state.  All matrix products are bf16 x bf16 with fp32 accumulation.
#include <algorithm>

#include "common.cuh"

namespace ti {

constexpr int kC = 64;   // chunk length

struct GdnChunkParams {
  const __nv_bfloat16* proj;   // [T, ld]: q | k | v | z | b | a columns (per-rank head counts)
  const float* conv_w;         // [2*hk*DK + hv*DV, 4]
  const float* neg_a_exp;      // [hv]
  const float* dt_bias;        // [hv]
  const float* norm_w;         // [DV]
  void* state;                 // [slots, hv, DK, DV] fp32 or bf16
  __nv_bfloat16* conv_state;   // [slots, hv, 3, 2*DK + DV]
  const int* slots;            // [S]
  const int* cu;               // [S+1] token offsets
  __nv_bfloat16* out;          // [T, hv*DV]
  const int* snap_rel;         // [S, NS] snapshot after this many tokens of the step (<= 0: unused), or nullptr
  const int* snap_idx;         // [S, NS] entry of the snapshot buffers
  float* snap_state;           // [entries, hv, DK, DV]
  __nv_bfloat16* snap_conv;    // [entries, hv, 3, 2*DK + DV]
  // chunk table (chunks of a sequence are consecutive and in order)
  const int* ck_seq;           // [nc]
  const int* ck_tok0;          // [nc] first flat token
  const int* ck_ntok;          // [nc] 1..64
  const int* ck_snap;          // [nc] snapshot entry to write after this chunk, or -1
  const int* seq_ck;           // [S+1] chunk range of every sequence
  // workspace, fragment order (index ch = chunk * hv + v-head)
  uint4* wf;                   // [ch][4 m-tiles][DK/16 k-tiles][32 lanes]   A fragments of w   (64 x DK)
  uint4* qf;                   // the same for q exp(g) DK^-1/2
  uint4* mf;                   // [ch][4][4][32]                              A fragments of the masked q k^T (64 x 64)
  uint2* kf;                   // [ch][4 k-tiles][DK/8 n-tiles][32]          B fragments of k exp(g_C - g) (64 x DK)
  float* u;                    // [ch][64][DV]
  float* gamma;                // [ch] exp(g_C)
  int ld, hk, hv, num_snap, nc;
  float eps;
};

TI_DEVICE uint32_t lds32(const __nv_bfloat16* p) { return *reinterpret_cast<const uint32_t*>(p); }
TI_DEVICE float bf(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// ---------------------------------------------------------------------------------------------------------------
// Prepare: one CTA per (chunk, v-head), 8 warps.
template <int DK, int DV>
struct PrepSmem {
  static constexpr int QS = DK + 8;      // bf16 row stride of the normalised q / k (conflict-free fragment loads)
  static constexpr int TS = kC + 8;      // bf16 row stride of token-minor arrays
  static constexpr size_t kBytes = (size_t)2 * kC * QS * 2 + (size_t)(DV + DK) * TS * 2 + (size_t)kC * TS * 2 +
                                   (size_t)kC * 65 * 4 + 32 * 33 * 4 + 4 * kC * 4;
};

template <int DK, int DV>
__global__ void __launch_bounds__(256) gdn_chunk_prepare_kernel(const __grid_constant__ GdnChunkParams p) {
  using SM = PrepSmem<DK, DV>;
  constexpr int QS = SM::QS, TS = SM::TS, KT = DK / 16, NCH = 2 * DK + DV;
  constexpr int EQ = DK / 32, EV = DV / 32;       // channels per lane in the conv stage
  extern __shared__ __align__(16) uint8_t smem[];
  __nv_bfloat16* qn = reinterpret_cast<__nv_bfloat16*>(smem);     // [64][QS]  q / |q| / sqrt(DK)
  __nv_bfloat16* kn = qn + kC * QS;                               // [64][QS]  k / |k|
  __nv_bfloat16* bvT = kn + kC * QS;                              // [DV][TS]  (b v)^T
  __nv_bfloat16* bkT = bvT + DV * TS;                             // [DK][TS]  (b exp(g) k)^T
  __nv_bfloat16* Xb = bkT + DK * TS;                              // [64][TS]  X in bf16
  float* Lm = reinterpret_cast<float*>(Xb + kC * TS);             // [64][65]  L, then X
  float* Tm = Lm + kC * 65;                                       // [32][33]
  float* gc = Tm + 32 * 33;                                       // [64] cumulative log decay
  float* bet = gc + kC;                                           // [64]
  float* eg = bet + kC;                                           // [64] exp(gc)
  float* egl = eg + kC;                                           // [64] exp(g_C - gc)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int ci = blockIdx.x, vh = blockIdx.y;
  const int kh = vh / (p.hv / p.hk);
  const int s = p.ck_seq[ci], tok0 = p.ck_tok0[ci], n = p.ck_ntok[ci];
  const int seq_t0 = p.cu[s];
  const int slot = p.slots[s];
  const size_t ch = (size_t)ci * p.hv + vh;
  const int bcol = 2 * p.hk * DK + 2 * p.hv * DV + vh, acol = bcol + p.hv;
  pdl_trigger();
  pdl_wait();

  // ---- A. gates: log decay, beta, inclusive scan over the chunk (warp 0; lane -> tokens lane, lane + 32)
  if (warp == 0) {
    const float neg_a = p.neg_a_exp[vh], dtb = p.dt_bias[vh];
    float gl[2], bb[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int j = lane + 32 * h;
      gl[h] = 0.f;
      bb[h] = 0.f;
      if (j < n) {
        const __nv_bfloat16* row = p.proj + (size_t)(tok0 + j) * p.ld;
        const float a = bf(row + acol) + dtb;
        const float sp = a > 20.f ? a : log1pf(__expf(a));
        gl[h] = neg_a * sp;
        bb[h] = sigmoid_f(bf(row + bcol));
      }
    }
    float c0 = gl[0], c1 = gl[1];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float a0 = __shfl_up_sync(0xffffffffu, c0, o), a1 = __shfl_up_sync(0xffffffffu, c1, o);
      if (lane >= o) { c0 += a0; c1 += a1; }
    }
    c1 += __shfl_sync(0xffffffffu, c0, 31);
    const float glast = __shfl_sync(0xffffffffu, c1, 31);
    gc[lane] = c0; gc[lane + 32] = c1;
    bet[lane] = bb[0]; bet[lane + 32] = bb[1];
    eg[lane] = __expf(c0); eg[lane + 32] = __expf(c1);
    egl[lane] = __expf(glast - c0); egl[lane + 32] = __expf(glast - c1);
    if (lane == 0) p.gamma[ch] = __expf(glast);
  }
  // conv taps of this lane's channels (lane -> EQ consecutive q and k channels, EV consecutive v channels)
  int colq[EQ], colv[EV];
  float4 wq[EQ], wk[EQ], wv[EV];
#pragma unroll
  for (int e = 0; e < EQ; ++e) {
    colq[e] = kh * DK + lane * EQ + e;
    wq[e] = *reinterpret_cast<const float4*>(p.conv_w + (size_t)colq[e] * 4);
    wk[e] = *reinterpret_cast<const float4*>(p.conv_w + (size_t)(p.hk * DK + colq[e]) * 4);
  }
#pragma unroll
  for (int e = 0; e < EV; ++e) {
    colv[e] = 2 * p.hk * DK + vh * DV + lane * EV + e;
    wv[e] = *reinterpret_cast<const float4*>(p.conv_w + (size_t)colv[e] * 4);
  }
  __syncthreads();

  // ---- B. causal conv + SiLU, q / k norms: a warp per token
  const __nv_bfloat16* hist = p.conv_state + ((size_t)slot * p.hv + vh) * 3 * NCH;
  const float qscale = rsqrtf((float)DK);
  for (int j = warp; j < kC; j += 8) {
    float yq[EQ], yk[EQ], yv[EV];
#pragma unroll
    for (int e = 0; e < EQ; ++e) yq[e] = yk[e] = 0.f;
#pragma unroll
    for (int e = 0; e < EV; ++e) yv[e] = 0.f;
    if (j < n) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int ti = tok0 + j - 3 + i;                  // flat token whose raw input feeds tap i
        const __nv_bfloat16* row = p.proj + (size_t)ti * p.ld;
        const bool from_hist = ti < seq_t0;
        const __nv_bfloat16* hrow = hist + (size_t)(ti - seq_t0 + 3) * NCH;
#pragma unroll
        for (int e = 0; e < EQ; ++e) {
          const float xq = from_hist ? bf(hrow + lane * EQ + e) : bf(row + colq[e]);
          const float xk = from_hist ? bf(hrow + DK + lane * EQ + e) : bf(row + p.hk * DK + colq[e]);
          const float cq = i == 0 ? wq[e].x : (i == 1 ? wq[e].y : (i == 2 ? wq[e].z : wq[e].w));
          const float ck = i == 0 ? wk[e].x : (i == 1 ? wk[e].y : (i == 2 ? wk[e].z : wk[e].w));
          yq[e] += cq * xq;
          yk[e] += ck * xk;
        }
#pragma unroll
        for (int e = 0; e < EV; ++e) {
          const float xv = from_hist ? bf(hrow + 2 * DK + lane * EV + e) : bf(row + colv[e]);
          const float cv = i == 0 ? wv[e].x : (i == 1 ? wv[e].y : (i == 2 ? wv[e].z : wv[e].w));
          yv[e] += cv * xv;
        }
      }
      float sq = 0.f, sk = 0.f;
#pragma unroll
      for (int e = 0; e < EQ; ++e) {
        yq[e] = silu_f(yq[e]);
        yk[e] = silu_f(yk[e]);
        sq += yq[e] * yq[e];
        sk += yk[e] * yk[e];
      }
#pragma unroll
      for (int e = 0; e < EV; ++e) yv[e] = silu_f(yv[e]);
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      const float qf_ = rsqrtf(sq + 1e-6f) * qscale, kf_ = rsqrtf(sk + 1e-6f);
#pragma unroll
      for (int e = 0; e < EQ; ++e) { yq[e] *= qf_; yk[e] *= kf_; }
    }
    const float b = bet[j], bge = b * eg[j];
#pragma unroll
    for (int e = 0; e < EQ; ++e) {
      qn[j * QS + lane * EQ + e] = __float2bfloat16_rn(yq[e]);
      kn[j * QS + lane * EQ + e] = __float2bfloat16_rn(yk[e]);
      bkT[(lane * EQ + e) * TS + j] = __float2bfloat16_rn(bge * yk[e]);
    }
#pragma unroll
    for (int e = 0; e < EV; ++e) bvT[(lane * EV + e) * TS + j] = __float2bfloat16_rn(b * yv[e]);
  }
  __syncthreads();

  // ---- C. k k^T and q k^T (64 x 64 each): warp -> m-tile (warp & 3), four n-tiles (warp >> 2)
  {
    const int mt = warp & 3, half = warp >> 2;
    float akk[4][4], aqk[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) akk[a][b] = aqk[a][b] = 0.f;
    const __nv_bfloat16* kr0 = kn + (16 * mt + g) * QS + 2 * t;
    const __nv_bfloat16* qr0 = qn + (16 * mt + g) * QS + 2 * t;
#pragma unroll
    for (int kt = 0; kt < KT; ++kt) {
      const uint32_t k0 = lds32(kr0 + 16 * kt), k1 = lds32(kr0 + 8 * QS + 16 * kt), k2 = lds32(kr0 + 16 * kt + 8),
                     k3 = lds32(kr0 + 8 * QS + 16 * kt + 8);
      const uint32_t q0 = lds32(qr0 + 16 * kt), q1 = lds32(qr0 + 8 * QS + 16 * kt), q2 = lds32(qr0 + 16 * kt + 8),
                     q3 = lds32(qr0 + 8 * QS + 16 * kt + 8);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const __nv_bfloat16* br = kn + (8 * (4 * half + c) + g) * QS + 16 * kt + 2 * t;
        const uint32_t b0 = lds32(br), b1 = lds32(br + 8);
        mma_bf16_16816(akk[c], k0, k1, k2, k3, b0, b1);
        mma_bf16_16816(aqk[c], q0, q1, q2, q3, b0, b1);
      }
    }
    const int i0 = 16 * mt + g, i1 = i0 + 8;
    const float g0 = gc[i0], g1 = gc[i1], be0 = bet[i0], be1 = bet[i1];
    uint32_t mpk[4][2];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int j0 = 8 * (4 * half + c) + 2 * t, j1 = j0 + 1;
      const float gj0 = gc[j0], gj1 = gc[j1];
      const float d00 = i0 >= j0 ? __expf(g0 - gj0) : 0.f, d01 = i0 >= j1 ? __expf(g0 - gj1) : 0.f;
      const float d10 = i1 >= j0 ? __expf(g1 - gj0) : 0.f, d11 = i1 >= j1 ? __expf(g1 - gj1) : 0.f;
      Lm[i0 * 65 + j0] = i0 > j0 ? be0 * akk[c][0] * d00 : 0.f;
      Lm[i0 * 65 + j1] = i0 > j1 ? be0 * akk[c][1] * d01 : 0.f;
      Lm[i1 * 65 + j0] = i1 > j0 ? be1 * akk[c][2] * d10 : 0.f;
      Lm[i1 * 65 + j1] = i1 > j1 ? be1 * akk[c][3] * d11 : 0.f;
      mpk[c][0] = pack_bf16(aqk[c][0] * d00, aqk[c][1] * d01);
      mpk[c][1] = pack_bf16(aqk[c][2] * d10, aqk[c][3] * d11);
    }
    // accumulator tiles (2kt, 2kt+1) -> A fragment of k-tile kt
#pragma unroll
    for (int kk = 0; kk < 2; ++kk)
      p.mf[((ch * 4 + mt) * 4 + 2 * half + kk) * 32 + lane] =
          make_uint4(mpk[2 * kk][0], mpk[2 * kk][1], mpk[2 * kk + 1][0], mpk[2 * kk + 1][1]);
  }
  __syncthreads();

  // ---- D. X = (I + L)^-1, blocked: 16 x 16 diagonal blocks by forward substitution (a column per lane),
  //         then X21 = -X22 (L21 X11) for the 16- and the 32-blocks.  In place in Lm.
  if (warp < 4) {
    const int b0 = 16 * warp, jj = lane & 15;
    for (int ii = 0; ii < 16; ++ii) {
      float acc = ii == jj ? 1.f : 0.f;
      if (lane < 16 && jj < ii)
        for (int m = jj; m < ii; ++m) acc -= Lm[(b0 + ii) * 65 + b0 + m] * Lm[(b0 + m) * 65 + b0 + jj];
      __syncwarp();
      if (lane < 16) Lm[(b0 + ii) * 65 + b0 + jj] = jj <= ii ? acc : 0.f;
      __syncwarp();
    }
  }
  __syncthreads();
  for (int sz = 16; sz <= 32; sz *= 2) {
    const int nblk = kC / (2 * sz);                         // pairs at this level
    // T = L21 X11
    for (int idx = tid; idx < nblk * sz * sz; idx += 256) {
      const int bq = idx / (sz * sz), r = (idx / sz) % sz, c = idx % sz;
      const int base = bq * 2 * sz;
      float acc = 0.f;
      for (int m = c; m < sz; ++m) acc += Lm[(base + sz + r) * 65 + base + m] * Lm[(base + m) * 65 + base + c];
      Tm[(bq * sz + r) * 33 + c] = acc;
    }
    __syncthreads();
    // X21 = -X22 T
    for (int idx = tid; idx < nblk * sz * sz; idx += 256) {
      const int bq = idx / (sz * sz), r = (idx / sz) % sz, c = idx % sz;
      const int base = bq * 2 * sz;
      float acc = 0.f;
      for (int m = 0; m <= r; ++m) acc += Lm[(base + sz + r) * 65 + base + sz + m] * Tm[(bq * sz + m) * 33 + c];
      Lm[(base + sz + r) * 65 + base + c] = -acc;
    }
    __syncthreads();
  }
  for (int idx = tid; idx < kC * kC; idx += 256) {
    const int r = idx >> 6, c = idx & 63;
    Xb[r * TS + c] = __float2bfloat16_rn(Lm[r * 65 + c]);
  }
  __syncthreads();

  // ---- E. u = X (b v), w = X (b exp(g) k): warp -> m-tile (warp & 3), half of the columns (warp >> 2)
  {
    const int mt = warp & 3, half = warp >> 2;
    uint32_t xa[4][4];
    const __nv_bfloat16* xr = Xb + (16 * mt + g) * TS + 2 * t;
#pragma unroll
    for (int kt = 0; kt < 4; ++kt) {
      xa[kt][0] = lds32(xr + 16 * kt);
      xa[kt][1] = lds32(xr + 8 * TS + 16 * kt);
      xa[kt][2] = lds32(xr + 16 * kt + 8);
      xa[kt][3] = lds32(xr + 8 * TS + 16 * kt + 8);
    }
    float* urow0 = p.u + (ch * kC + 16 * mt + g) * DV;
#pragma unroll 2
    for (int c = 0; c < DV / 16; ++c) {
      const int nt = half * (DV / 16) + c;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kt = 0; kt < 4; ++kt) {
        const __nv_bfloat16* br = bvT + (8 * nt + g) * TS + 16 * kt + 2 * t;
        mma_bf16_16816(acc, xa[kt][0], xa[kt][1], xa[kt][2], xa[kt][3], lds32(br), lds32(br + 8));
      }
      *reinterpret_cast<float2*>(urow0 + 8 * nt + 2 * t) = make_float2(acc[0], acc[1]);
      *reinterpret_cast<float2*>(urow0 + 8 * DV + 8 * nt + 2 * t) = make_float2(acc[2], acc[3]);
    }
#pragma unroll 2
    for (int c = 0; c < KT / 2; ++c) {
      const int kt2 = half * (KT / 2) + c;                    // k-tile of w = pair of accumulator n-tiles
      float acc[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
#pragma unroll
        for (int kt = 0; kt < 4; ++kt) {
          const __nv_bfloat16* br = bkT + (8 * (2 * kt2 + h) + g) * TS + 16 * kt + 2 * t;
          mma_bf16_16816(acc[h], xa[kt][0], xa[kt][1], xa[kt][2], xa[kt][3], lds32(br), lds32(br + 8));
        }
      }
      p.wf[((ch * 4 + mt) * KT + kt2) * 32 + lane] = make_uint4(pack_bf16(acc[0][0], acc[0][1]), pack_bf16(acc[0][2], acc[0][3]),
                                                               pack_bf16(acc[1][0], acc[1][1]), pack_bf16(acc[1][2], acc[1][3]));
    }
  }
  // ---- F. q exp(g) as A fragments, k exp(g_C - g) as B fragments
  for (int idx = tid; idx < 4 * KT * 32; idx += 256) {
    const int ln = idx & 31, kt = (idx >> 5) % KT, mt = idx / (32 * KT);
    const int gg = ln >> 2, tt = ln & 3;
    const int r0 = 16 * mt + gg, r1 = r0 + 8, c0 = 16 * kt + 2 * tt;
    const float e0 = eg[r0], e1 = eg[r1];
    const __nv_bfloat16* a = qn + r0 * QS + c0;
    const __nv_bfloat16* b = qn + r1 * QS + c0;
    p.qf[(ch * 4 * KT) * 32 + idx] = make_uint4(pack_bf16(bf(a) * e0, bf(a + 1) * e0), pack_bf16(bf(b) * e1, bf(b + 1) * e1),
                                                pack_bf16(bf(a + 8) * e0, bf(a + 9) * e0), pack_bf16(bf(b + 8) * e1, bf(b + 9) * e1));
  }
  for (int idx = tid; idx < 4 * (DK / 8) * 32; idx += 256) {
    const int ln = idx & 31, nt = (idx >> 5) % (DK / 8), kt = idx / (32 * (DK / 8));
    const int gg = ln >> 2, tt = ln & 3;
    const int r0 = 16 * kt + 2 * tt, d = 8 * nt + gg;
    p.kf[(ch * 4 * (DK / 8)) * 32 + idx] =
        make_uint2(pack_bf16(bf(kn + r0 * QS + d) * egl[r0], bf(kn + (r0 + 1) * QS + d) * egl[r0 + 1]),
                   pack_bf16(bf(kn + (r0 + 8) * QS + d) * egl[r0 + 8], bf(kn + (r0 + 9) * QS + d) * egl[r0 + 9]));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Scan: one CTA (4 warps) per (v-head, 32 state columns, sequence).
template <typename ST> TI_DEVICE float ldst(const ST* p);
template <> TI_DEVICE float ldst<float>(const float* p) { return *p; }
template <> TI_DEVICE float ldst<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename ST> TI_DEVICE void stst(ST* p, float v);
template <> TI_DEVICE void stst<float>(float* p, float v) { *p = v; }
template <> TI_DEVICE void stst<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int DK, int DV, typename ST>
__global__ void __launch_bounds__(128) gdn_chunk_scan_kernel(const __grid_constant__ GdnChunkParams p) {
  constexpr int DVB = 32, NB = DV / DVB, KT = DK / 16, NTV = DVB / 8, NTW = DK / 32, MTS = DVB / 16;
  constexpr int SS = DK + 8, VS = kC + 8;
  __shared__ __align__(16) __nv_bfloat16 Sb[DVB * SS];          // S^T (bf16): row = state column, pairs along dk
  __shared__ __align__(16) __nv_bfloat16 vnT[2][DVB * VS];      // v_new^T (bf16), double-buffered by chunk

  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int vh = blockIdx.x / NB, dv0 = (blockIdx.x % NB) * DVB, s = blockIdx.y;
  const int slot = p.slots[s];
  ST* Sp = static_cast<ST*>(p.state) + ((size_t)slot * p.hv + vh) * DK * DV;
  const int dk0 = w * (DK / 4);                                  // this warp's slice of dk in the state update

  // state slice as S^T accumulator fragments: sT[mt][j] covers rows (state columns) 16mt + g (+8), dk = dk0 + 8j + 2t (+1)
  float sT[MTS][NTW][4];
#pragma unroll
  for (int mt = 0; mt < MTS; ++mt)
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      const int d = dk0 + 8 * j + 2 * t, c = dv0 + 16 * mt + g;
      sT[mt][j][0] = ldst<ST>(Sp + (size_t)d * DV + c);
      sT[mt][j][1] = ldst<ST>(Sp + (size_t)(d + 1) * DV + c);
      sT[mt][j][2] = ldst<ST>(Sp + (size_t)d * DV + c + 8);
      sT[mt][j][3] = ldst<ST>(Sp + (size_t)(d + 1) * DV + c + 8);
    }
  auto publish_state = [&]() {
#pragma unroll
    for (int mt = 0; mt < MTS; ++mt)
#pragma unroll
      for (int j = 0; j < NTW; ++j) {
        const int d = dk0 + 8 * j + 2 * t;
        *reinterpret_cast<uint32_t*>(Sb + (16 * mt + g) * SS + d) = pack_bf16(sT[mt][j][0], sT[mt][j][1]);
        *reinterpret_cast<uint32_t*>(Sb + (16 * mt + g + 8) * SS + d) = pack_bf16(sT[mt][j][2], sT[mt][j][3]);
      }
  };
  publish_state();
  pdl_trigger();
  pdl_wait();                                                    // the operands come from the prepare kernel
  __syncthreads();

  const int c_lo = p.seq_ck[s], c_hi = p.seq_ck[s + 1];
  for (int ci = c_lo; ci < c_hi; ++ci) {
    const size_t ch = (size_t)ci * p.hv + vh;
    const int ntok = p.ck_ntok[ci], tok0 = p.ck_tok0[ci];
    __nv_bfloat16* vT = vnT[(ci - c_lo) & 1];
    // ---- v_new rows of this warp = u - w S ; o rows = (q exp g) S
    float av[NTV][4], ao[NTV][4];
    const float* urow = p.u + (ch * kC + 16 * w + g) * DV + dv0 + 2 * t;
#pragma unroll
    for (int nt = 0; nt < NTV; ++nt) {
      const float2 u0 = *reinterpret_cast<const float2*>(urow + 8 * nt);
      const float2 u1 = *reinterpret_cast<const float2*>(urow + 8 * DV + 8 * nt);
      av[nt][0] = u0.x; av[nt][1] = u0.y; av[nt][2] = u1.x; av[nt][3] = u1.y;
      ao[nt][0] = ao[nt][1] = ao[nt][2] = ao[nt][3] = 0.f;
    }
    const uint4* wfp = p.wf + ((ch * 4 + w) * KT) * 32 + lane;
    const uint4* qfp = p.qf + ((ch * 4 + w) * KT) * 32 + lane;
#pragma unroll
    for (int kt = 0; kt < KT; ++kt) {
      uint4 aw = __ldg(wfp + kt * 32);
      const uint4 aq = __ldg(qfp + kt * 32);
      aw.x ^= 0x80008000u; aw.y ^= 0x80008000u; aw.z ^= 0x80008000u; aw.w ^= 0x80008000u;     // -w
#pragma unroll
      for (int nt = 0; nt < NTV; ++nt) {
        const __nv_bfloat16* br = Sb + (8 * nt + g) * SS + 16 * kt + 2 * t;
        const uint32_t b0 = lds32(br), b1 = lds32(br + 8);
        mma_bf16_16816(av[nt], aw.x, aw.y, aw.z, aw.w, b0, b1);
        mma_bf16_16816(ao[nt], aq.x, aq.y, aq.z, aq.w, b0, b1);
      }
    }
#pragma unroll
    for (int nt = 0; nt < NTV; ++nt) {
      const int c = 8 * nt + 2 * t, r = 16 * w + g;
      vT[c * VS + r] = __float2bfloat16_rn(av[nt][0]);
      vT[(c + 1) * VS + r] = __float2bfloat16_rn(av[nt][1]);
      vT[c * VS + r + 8] = __float2bfloat16_rn(av[nt][2]);
      vT[(c + 1) * VS + r + 8] = __float2bfloat16_rn(av[nt][3]);
    }
    __syncthreads();
    // ---- o rows += (masked q k^T) v_new : the k-tiles above the diagonal are zero
    const uint4* mfp = p.mf + ((ch * 4 + w) * 4) * 32 + lane;
    for (int kt = 0; kt <= w; ++kt) {
      const uint4 am = __ldg(mfp + kt * 32);
#pragma unroll
      for (int nt = 0; nt < NTV; ++nt) {
        const __nv_bfloat16* br = vT + (8 * nt + g) * VS + 16 * kt + 2 * t;
        mma_bf16_16816(ao[nt], am.x, am.y, am.z, am.w, lds32(br), lds32(br + 8));
      }
    }
    {
      const int r0 = 16 * w + g, r1 = r0 + 8;
      __nv_bfloat16* o0 = p.out + (size_t)(tok0 + r0) * p.hv * DV + vh * DV + dv0 + 2 * t;
      __nv_bfloat16* o1 = p.out + (size_t)(tok0 + r1) * p.hv * DV + vh * DV + dv0 + 2 * t;
#pragma unroll
      for (int nt = 0; nt < NTV; ++nt) {
        if (r0 < ntok) *reinterpret_cast<uint32_t*>(o0 + 8 * nt) = pack_bf16(ao[nt][0], ao[nt][1]);
        if (r1 < ntok) *reinterpret_cast<uint32_t*>(o1 + 8 * nt) = pack_bf16(ao[nt][2], ao[nt][3]);
      }
    }
    // ---- S^T slice <- gamma S^T + v_new^T (k exp(g_C - g))
    const float gam = p.gamma[ch];
#pragma unroll
    for (int mt = 0; mt < MTS; ++mt)
#pragma unroll
      for (int j = 0; j < NTW; ++j) {
        sT[mt][j][0] *= gam; sT[mt][j][1] *= gam; sT[mt][j][2] *= gam; sT[mt][j][3] *= gam;
      }
    const uint2* kfp = p.kf + (ch * 4 * (DK / 8)) * 32 + lane;
#pragma unroll
    for (int kt = 0; kt < 4; ++kt) {
      uint2 kb[NTW];
#pragma unroll
      for (int j = 0; j < NTW; ++j) kb[j] = __ldg(kfp + (kt * (DK / 8) + w * NTW + j) * 32);
#pragma unroll
      for (int mt = 0; mt < MTS; ++mt) {
        const __nv_bfloat16* ar = vT + (16 * mt + g) * VS + 16 * kt + 2 * t;
        const uint32_t a0 = lds32(ar), a1 = lds32(ar + 8 * VS), a2 = lds32(ar + 8), a3 = lds32(ar + 8 * VS + 8);
#pragma unroll
        for (int j = 0; j < NTW; ++j) mma_bf16_16816(sT[mt][j], a0, a1, a2, a3, kb[j].x, kb[j].y);
      }
    }
    publish_state();
    const int snap = p.ck_snap[ci];
    if (snap >= 0) {
      float* dst = p.snap_state + ((size_t)snap * p.hv + vh) * DK * DV;
#pragma unroll
      for (int mt = 0; mt < MTS; ++mt)
#pragma unroll
        for (int j = 0; j < NTW; ++j) {
          const int d = dk0 + 8 * j + 2 * t, c = dv0 + 16 * mt + g;
          dst[(size_t)d * DV + c] = sT[mt][j][0];
          dst[(size_t)(d + 1) * DV + c] = sT[mt][j][1];
          dst[(size_t)d * DV + c + 8] = sT[mt][j][2];
          dst[(size_t)(d + 1) * DV + c + 8] = sT[mt][j][3];
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int mt = 0; mt < MTS; ++mt)
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      const int d = dk0 + 8 * j + 2 * t, c = dv0 + 16 * mt + g;
      stst<ST>(Sp + (size_t)d * DV + c, sT[mt][j][0]);
      stst<ST>(Sp + (size_t)(d + 1) * DV + c, sT[mt][j][1]);
      stst<ST>(Sp + (size_t)d * DV + c + 8, sT[mt][j][2]);
      stst<ST>(Sp + (size_t)(d + 1) * DV + c + 8, sT[mt][j][3]);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Finish: gated RMSNorm over the head * silu(z), in place on the un-normalised output.  A warp per (token, v-head).
template <int DV>
__global__ void __launch_bounds__(256) gdn_chunk_finish_kernel(const __grid_constant__ GdnChunkParams p, int T, int DK) {
  constexpr int E = DV / 32;
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();
  if (item >= T * p.hv) return;
  const int tok = item / p.hv, vh = item - tok * p.hv;
  __nv_bfloat16* o = p.out + (size_t)tok * p.hv * DV + vh * DV + lane * E;
  const __nv_bfloat16* z = p.proj + (size_t)tok * p.ld + 2 * p.hk * DK + p.hv * DV + vh * DV + lane * E;
  float v[E], ss = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    v[e] = bf(o + e);
    ss += v[e] * v[e];
  }
  ss = warp_sum(ss);
  const float rr = rsqrtf(ss / (float)DV + p.eps);
#pragma unroll
  for (int e = 0; e < E; ++e) o[e] = __float2bfloat16_rn(v[e] * rr * p.norm_w[lane * E + e] * silu_f(bf(z + e)));
}

// Conv history after the step (z = 0) and at the snapshot points (z = 1 + point): the raw inputs of the last three
// tokens before that position.  Grid (S, hv, 1 + num_snap).  Snapshot points lie at least three tokens into the
// step (they are block-aligned), so only the z = 0 blocks ever read the old history they also overwrite.
__global__ void __launch_bounds__(128) gdn_conv_tail_kernel(const __grid_constant__ GdnChunkParams p, int DK, int DV) {
  const int s = blockIdx.x, vh = blockIdx.y, z = blockIdx.z;
  const int NCH = 2 * DK + DV;
  const int kh = vh / (p.hv / p.hk);
  const int t0 = p.cu[s], t1 = p.cu[s + 1];
  int n = t1 - t0;
  __nv_bfloat16* hist = p.conv_state + ((size_t)p.slots[s] * p.hv + vh) * 3 * NCH;
  __nv_bfloat16* dst = hist;
  if (z > 0) {
    if (p.snap_rel == nullptr) return;
    const int rel = p.snap_rel[s * p.num_snap + z - 1];
    if (rel <= 0 || rel > n) return;
    n = rel;
    dst = p.snap_conv + ((size_t)p.snap_idx[s * p.num_snap + z - 1] * p.hv + vh) * 3 * NCH;
  }
  for (int c = threadIdx.x; c < NCH; c += blockDim.x) {
    const int col = c < DK ? kh * DK + c : (c < 2 * DK ? p.hk * DK + kh * DK + (c - DK) : 2 * p.hk * DK + vh * DV + (c - 2 * DK));
    __nv_bfloat16 v[3];
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int ti = n - 3 + j;                               // token of the step (negative: older than the step)
      v[j] = ti >= 0 ? p.proj[(size_t)(t0 + ti) * p.ld + col] : hist[(size_t)(3 + ti) * NCH + c];
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) dst[(size_t)j * NCH + c] = v[j];
  }
}

template <int DK, int DV>
static int launch_chunked(const GdnChunkParams& p, int S, int T, int state_bf16, cudaStream_t st) {
  auto prep = gdn_chunk_prepare_kernel<DK, DV>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(prep, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PrepSmem<DK, DV>::kBytes);
    configured = true;
  }
  cudaError_t e = launch_kernel(prep, dim3(p.nc, p.hv), dim3(256), PrepSmem<DK, DV>::kBytes, st, true, p);
  if (e != cudaSuccess) return (int)e;
  const dim3 sgrid(p.hv * (DV / 32), S);
  if (state_bf16) e = launch_kernel(gdn_chunk_scan_kernel<DK, DV, __nv_bfloat16>, sgrid, dim3(128), 0, st, true, p);
  else e = launch_kernel(gdn_chunk_scan_kernel<DK, DV, float>, sgrid, dim3(128), 0, st, true, p);
  if (e != cudaSuccess) return (int)e;
  e = launch_kernel(gdn_chunk_finish_kernel<DV>, dim3((T * p.hv + 7) / 8), dim3(256), 0, st, true, p, T, DK);
  if (e != cudaSuccess) return (int)e;
  // not a programmatic launch: it overwrites the conv history the prepare kernel reads
  gdn_conv_tail_kernel<<<dim3(S, p.hv, 1 + (p.snap_rel != nullptr ? p.num_snap : 0)), 128, 0, st>>>(p, DK, DV);
  return (int)cudaGetLastError();
}

}  // namespace ti

extern "C" {

int ti_gdn_chunk_params_size() { return (int)sizeof(ti::GdnChunkParams); }

// Bytes of workspace per (chunk, v-head): wf, qf, mf, kf, u, gamma (in this order, see GdnChunkParams).
int ti_gdn_chunk_ws_bytes(int dk, int dv, int which) {
  switch (which) {
    case 0: case 1: return 4 * (dk / 16) * 32 * 16;
    case 2: return 4 * 4 * 32 * 16;
    case 3: return 4 * (dk / 8) * 32 * 8;
    case 4: return 64 * dv * 4;
    default: return 4;
  }
}

// Chunked prefill of the gated DeltaNet mixer for a flattened batch (see the file comment): prepare, scan, finish,
// conv tail.  `num_seqs` sequences, `T` tokens; the chunk table in `p` must cover every token exactly once.
int ti_gdn_chunked(const ti::GdnChunkParams* p, int num_seqs, int T, int dk, int dv, int state_bf16, void* stream) {
  if (num_seqs <= 0 || p->nc <= 0) return 0;
  if (p->hv % p->hk) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  if (dk == 128 && dv == 128) return ti::launch_chunked<128, 128>(*p, num_seqs, T, state_bf16, st);
  if (dk == 64 && dv == 64) return ti::launch_chunked<64, 64>(*p, num_seqs, T, state_bf16, st);
  return -3;
}

}  // extern "C"
