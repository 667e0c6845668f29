// Gated DeltaNet token mixer: causal depthwise conv1d + SiLU, q/k L2 normalisation, gates, the
// gated delta rule and the gated RMSNorm in ONE kernel that updates the recurrent state and the
// conv history in place inside their pool slots.
//
// Replaces, for decode, kernels/causal_conv1d.py:6-57 + kernels/deltanet_fused.py:10-684 and the
// state gather/scatter copies around them (model/qwen_36.py:151-156, 742-766); for prefill it
// replaces kernels/causal_conv1d.py:60-115 and the chunk kernel of
// kernels/gated_delta_rule_prefill.py:28-120, which drops the (v - S^T k) correction.  Here prefill
// runs the same exact recurrence token by token with the state held in registers, so a prompt
// processed in one piece, in chunks, or one token at a time gives the same state; everything that is not
// the recurrence itself (conv, norms, gates, output norm) is done for 16 tokens at a time.
//
// Mapping: one block per (v-head, sequence); thread = (column c of the state, quarter dg of the
// key dimension) with the four quarters of a column in adjacent lanes, so both matrix-vector
// products of a step reduce with two warp shuffles.  A state column never interacts with other
// columns, only the gated norm needs a block-wide sum.
//
// Conv history layout: [slot][v-head][3][2*DK + DV]; every v-head keeps its own copy of the q/k
// history of the key head it shares, so blocks never write memory another block reads.
#include "common.cuh"

namespace ti {

struct GdnParams {
  const __nv_bfloat16* proj;   // [T, ld]: q | k | v | z | b | a columns (per-rank head counts)
  const float* conv_w;         // [2*hk*DK + hv*DV, 4]
  const float* neg_a_exp;      // [hv]  -exp(A_log)
  const float* dt_bias;        // [hv]
  const float* norm_w;         // [DV]
  void* state;                 // [slots, hv, DK, DV]  fp32 or bf16
  __nv_bfloat16* conv_state;   // [slots, hv, 3, 2*DK + DV]
  const int* slots;            // [S]
  const int* cu;               // [S+1] token offsets, or nullptr (one token per sequence)
  __nv_bfloat16* out;          // [T, hv*DV]
  const int* snap_rel;         // [S, NS] snapshot after this many tokens of the chunk (<=0: unused) or nullptr
  float* snap_state;           // [S, NS, hv, DK, DV]
  __nv_bfloat16* snap_conv;    // [S, NS, hv, 3, 2*DK + DV]
  int ld, hk, hv, num_snap;
  float eps;
};

template <typename ST> TI_DEVICE float ld_state(const ST* p);
template <> TI_DEVICE float ld_state<float>(const float* p) { return *p; }
template <> TI_DEVICE float ld_state<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename ST> TI_DEVICE void st_state(ST* p, float v);
template <> TI_DEVICE void st_state<float>(float* p, float v) { *p = v; }
template <> TI_DEVICE void st_state<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// Tokens are processed in tiles of kTT.  Per tile: (1) every conv channel runs its window over the tile's tokens
// (independent global loads, no synchronisation) and the per-token scalars (q/k norms, decay, beta) are worked
// out in parallel; (2) the recurrence walks the tile token by token out of shared memory: two matrix-vector
// products per token, reduced with warp shuffles, nothing else on the serial path; (3) the gated norm and the
// output are again parallel over the tile.  The arithmetic of a token does not depend on the tiling.
constexpr int kTT = 16;

template <int DK, int DV, typename ST>
__global__ void __launch_bounds__(DV * 4) gdn_kernel(const __grid_constant__ GdnParams p) {
  constexpr int DPT = DK / 4;           // state elements per thread
  constexpr int NCH = 2 * DK + DV;      // conv channels this block needs
  constexpr int NW = DV * 4 / 32;
  static_assert(NCH <= DV * 4, "one thread per conv channel");
  // q/k rows are padded by 4 floats per quarter so that the four quarters (lanes dg = 0..3 read different
  // quarters at the same time) fall into different banks
  constexpr int DKP = DK + 16;
  __shared__ __align__(16) float qs[kTT][DKP], ks[kTT][DKP], vs[kTT][DV];     // vs holds v, then the un-normalised output
  __shared__ float qn_s[kTT], kn_s[kTT], decay_s[kTT], beta_s[kTT], rr_s[kTT];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = tid >> 2, dg = tid & 3;
  const int vh = blockIdx.x, s = blockIdx.y;
  const int kh = vh / (p.hv / p.hk);
  // cu / slots are written by host copies that precede every kernel of the step; the recurrent state
  // and conv history were last written one step ago: all of this may be read before pdl_wait()
  const int t0 = p.cu ? p.cu[s] : s, t1 = p.cu ? p.cu[s + 1] : s + 1;
  const int slot = p.slots[s];

  ST* Sp = static_cast<ST*>(p.state) + ((size_t)slot * p.hv + vh) * DK * DV;
  float S[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) S[i] = ld_state<ST>(Sp + (size_t)(dg * DPT + i) * DV + c);

  // conv channel owned by this thread: column in `proj` and row of conv_w
  __nv_bfloat16* cs = p.conv_state + ((size_t)slot * p.hv + vh) * 3 * NCH;
  float x0 = 0.f, x1 = 0.f, x2 = 0.f, cw0 = 0.f, cw1 = 0.f, cw2 = 0.f, cw3 = 0.f;
  int col = 0;
  if (tid < NCH) {
    if (tid < DK) col = kh * DK + tid;
    else if (tid < 2 * DK) col = p.hk * DK + kh * DK + (tid - DK);
    else col = 2 * p.hk * DK + vh * DV + (tid - 2 * DK);
    const float4 w = *reinterpret_cast<const float4*>(p.conv_w + (size_t)col * 4);
    cw0 = w.x; cw1 = w.y; cw2 = w.z; cw3 = w.w;
    x0 = __bfloat162float(cs[tid]);
    x1 = __bfloat162float(cs[NCH + tid]);
    x2 = __bfloat162float(cs[2 * NCH + tid]);
  }
  const int zcol = 2 * p.hk * DK + p.hv * DV + vh * DV;
  const int bcol = 2 * p.hk * DK + 2 * p.hv * DV + vh;
  const int acol = bcol + p.hv;
  const float neg_a = p.neg_a_exp[vh], dtb = p.dt_bias[vh];
  const float qscale = rsqrtf((float)DK);
  pdl_trigger();
  pdl_wait();                                    // `proj` comes from the preceding projection kernel

  for (int tile0 = t0; tile0 < t1; tile0 += kTT) {
    const int nt = min(kTT, t1 - tile0);
    // ---- (1a) conv + SiLU of every channel over the tile
    if (tid < NCH) {
      float xin[kTT];
#pragma unroll
      for (int j = 0; j < kTT; ++j)
        xin[j] = j < nt ? __bfloat162float(p.proj[(size_t)(tile0 + j) * p.ld + col]) : 0.f;
#pragma unroll
      for (int j = 0; j < kTT; ++j) {
        if (j < nt) {
          const float x3 = xin[j];
          const float y = silu_f(cw0 * x0 + cw1 * x1 + cw2 * x2 + cw3 * x3);
          x0 = x1; x1 = x2; x2 = x3;
          if (tid < DK) qs[j][tid + 4 * (tid / DPT)] = y;
          else if (tid < 2 * DK) ks[j][(tid - DK) + 4 * ((tid - DK) / DPT)] = y;
          else vs[j][tid - 2 * DK] = y;
          if (p.snap_rel != nullptr) {             // conv window after token (tile0 + j)
            const int done = tile0 + j - t0 + 1;
            for (int q = 0; q < p.num_snap; ++q) {
              if (p.snap_rel[s * p.num_snap + q] != done) continue;
              __nv_bfloat16* dc = p.snap_conv + (((size_t)s * p.num_snap + q) * p.hv + vh) * 3 * NCH;
              dc[tid] = __float2bfloat16_rn(x0);
              dc[NCH + tid] = __float2bfloat16_rn(x1);
              dc[2 * NCH + tid] = __float2bfloat16_rn(x2);
            }
          }
        }
      }
    }
    __syncthreads();
    // ---- (1b) per-token scalars: a warp per token
    for (int j = warp; j < nt; j += NW) {
      const __nv_bfloat16* row = p.proj + (size_t)(tile0 + j) * p.ld;
      float sq = 0.f, sk = 0.f;
      for (int i = lane; i < DK; i += 32) {
        const float a = qs[j][i + 4 * (i / DPT)], b = ks[j][i + 4 * (i / DPT)];
        sq += a * a;
        sk += b * b;
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      if (lane == 0) {
        qn_s[j] = rsqrtf(sq + 1e-6f) * qscale;
        kn_s[j] = rsqrtf(sk + 1e-6f);
        const float a = __bfloat162float(row[acol]) + dtb;
        const float sp = a > 20.f ? a : log1pf(__expf(a));
        decay_s[j] = __expf(neg_a * sp);
        beta_s[j] = sigmoid_f(__bfloat162float(row[bcol]));
      }
    }
    __syncthreads();
    // ---- (2) the recurrence, token by token, out of shared memory
    for (int j = 0; j < nt; ++j) {
      const float decay = decay_s[j], kn = kn_s[j];
      const float* kj = ks[j] + dg * (DPT + 4);
      const float* qj = qs[j] + dg * (DPT + 4);
      float kv = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) { S[i] *= decay; kv += S[i] * kj[i]; }
      kv += __shfl_xor_sync(0xffffffffu, kv, 1);
      kv += __shfl_xor_sync(0xffffffffu, kv, 2);
      const float delta = (vs[j][c] - kv * kn) * beta_s[j];
      const float kd = kn * delta;
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) { S[i] += kj[i] * kd; o += S[i] * qj[i]; }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      __syncwarp();                                // all four lanes of the column have read vs[j][c]
      if (dg == 0) vs[j][c] = o * qn_s[j];
      if (p.snap_rel != nullptr) {
        const int done = tile0 + j - t0 + 1;
        for (int q = 0; q < p.num_snap; ++q) {
          if (p.snap_rel[s * p.num_snap + q] != done) continue;
          float* dst = p.snap_state + (((size_t)s * p.num_snap + q) * p.hv + vh) * DK * DV;
#pragma unroll
          for (int i = 0; i < DPT; ++i) dst[(size_t)(dg * DPT + i) * DV + c] = S[i];
        }
      }
    }
    __syncthreads();
    // ---- (3) gated RMSNorm * silu(z): a warp per token for the statistics, then all threads for the output
    for (int j = warp; j < nt; j += NW) {
      float o2 = 0.f;
      for (int i = lane; i < DV; i += 32) o2 += vs[j][i] * vs[j][i];
      o2 = warp_sum(o2);
      if (lane == 0) rr_s[j] = rsqrtf(o2 / (float)DV + p.eps);
    }
    __syncthreads();
    for (int e = tid; e < nt * DV; e += DV * 4) {
      const int j = e / DV, cc = e - j * DV;
      const size_t tok = (size_t)(tile0 + j);
      const float z = __bfloat162float(p.proj[tok * p.ld + zcol + cc]);
      p.out[tok * p.hv * DV + vh * DV + cc] = __float2bfloat16_rn(vs[j][cc] * rr_s[j] * p.norm_w[cc] * silu_f(z));
    }
    __syncthreads();                               // the tile buffers are reused
  }

#pragma unroll
  for (int i = 0; i < DPT; ++i) st_state<ST>(Sp + (size_t)(dg * DPT + i) * DV + c, S[i]);
  if (tid < NCH) {
    cs[tid] = __float2bfloat16_rn(x0);
    cs[NCH + tid] = __float2bfloat16_rn(x1);
    cs[2 * NCH + tid] = __float2bfloat16_rn(x2);
  }
}

}  // namespace ti

extern "C" {

int ti_gdn_params_size() { return (int)sizeof(ti::GdnParams); }

// state_bf16: 0 = fp32 state pool, 1 = bf16.  (dk, dv) must be (128,128) or (64,64).
int ti_gdn_step(const ti::GdnParams* p, int num_seqs, int dk, int dv, int state_bf16, void* stream) {
  if (num_seqs <= 0) return 0;
  if (p->hv % p->hk) return -2;
  dim3 grid(p->hv, num_seqs);
  cudaStream_t st = (cudaStream_t)stream;
  if (dk == 128 && dv == 128) {
    if (state_bf16) ti::launch_kernel(ti::gdn_kernel<128, 128, __nv_bfloat16>, grid, dim3(512), 0, st, true, *p);
    else ti::launch_kernel(ti::gdn_kernel<128, 128, float>, grid, dim3(512), 0, st, true, *p);
  } else if (dk == 64 && dv == 64) {
    if (state_bf16) ti::launch_kernel(ti::gdn_kernel<64, 64, __nv_bfloat16>, grid, dim3(256), 0, st, true, *p);
    else ti::launch_kernel(ti::gdn_kernel<64, 64, float>, grid, dim3(256), 0, st, true, *p);
  } else {
    return -3;
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
