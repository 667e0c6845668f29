// Gated DeltaNet token mixer: causal depthwise conv1d + SiLU, q/k L2 normalisation, gates, the
// gated delta rule and the gated RMSNorm in ONE kernel that updates the recurrent state and the
// conv history in place inside their pool slots.
//
// Replaces, for decode, kernels/causal_conv1d.py:6-57 + kernels/deltanet_fused.py:10-684 and the
// state gather/scatter copies around them (model/qwen_36.py:151-156, 742-766); for prefill it
// replaces kernels/causal_conv1d.py:60-115 and the chunk kernel of
// kernels/gated_delta_rule_prefill.py:28-120, which drops the (v - S^T k) correction.  Here prefill
// runs the same exact recurrence token by token with the state held in registers, so a prompt
// processed in one piece, in chunks, or one token at a time gives the same state.
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

template <int DK, int DV, typename ST>
__global__ void __launch_bounds__(DV * 4) gdn_kernel(const __grid_constant__ GdnParams p) {
  constexpr int DPT = DK / 4;           // state elements per thread
  constexpr int NCH = 2 * DK + DV;      // conv channels this block needs
  constexpr int NW = DV * 4 / 32;
  static_assert(NCH <= DV * 4, "one thread per conv channel");
  __shared__ float qs[DK], ks[DK], vs[DV], red[NW];

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
  const float nw = p.norm_w[c];
  const float qscale = rsqrtf((float)DK);
  pdl_trigger();
  pdl_wait();                                    // `proj` comes from the preceding projection kernel

  for (int tok = t0; tok < t1; ++tok) {
    const __nv_bfloat16* row = p.proj + (size_t)tok * p.ld;
    if (tid < NCH) {
      const float x3 = __bfloat162float(row[col]);
      const float y = silu_f(cw0 * x0 + cw1 * x1 + cw2 * x2 + cw3 * x3);
      x0 = x1; x1 = x2; x2 = x3;
      if (tid < DK) qs[tid] = y;
      else if (tid < 2 * DK) ks[tid - DK] = y;
      else vs[tid - 2 * DK] = y;
    }
    __syncthreads();
    float sq = 0.f, sk = 0.f;
    for (int i = lane; i < DK; i += 32) { sq += qs[i] * qs[i]; sk += ks[i] * ks[i]; }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float qn = rsqrtf(sq + 1e-6f) * qscale, kn = rsqrtf(sk + 1e-6f);
    const float a = __bfloat162float(row[acol]) + dtb;
    const float sp = a > 20.f ? a : log1pf(__expf(a));
    const float decay = __expf(neg_a * sp);
    const float beta = sigmoid_f(__bfloat162float(row[bcol]));

    float kv = 0.f;
#pragma unroll
    for (int i = 0; i < DPT; ++i) { S[i] *= decay; kv += S[i] * ks[dg * DPT + i]; }
    kv += __shfl_xor_sync(0xffffffffu, kv, 1);
    kv += __shfl_xor_sync(0xffffffffu, kv, 2);
    const float delta = (vs[c] - kv * kn) * beta;
    const float kd = kn * delta;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DPT; ++i) { S[i] += ks[dg * DPT + i] * kd; o += S[i] * qs[dg * DPT + i]; }
    o += __shfl_xor_sync(0xffffffffu, o, 1);
    o += __shfl_xor_sync(0xffffffffu, o, 2);
    o *= qn;

    float o2 = dg == 0 ? o * o : 0.f;
    o2 = warp_sum(o2);
    if (lane == 0) red[warp] = o2;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) tot += red[w];
    const float rr = rsqrtf(tot / (float)DV + p.eps);
    if (dg == 0) {
      const float z = __bfloat162float(row[zcol + c]);
      p.out[(size_t)tok * p.hv * DV + vh * DV + c] = __float2bfloat16_rn(o * rr * nw * silu_f(z));
    }
    if (p.snap_rel != nullptr) {
      const int done = tok - t0 + 1;
      for (int j = 0; j < p.num_snap; ++j) {
        if (p.snap_rel[s * p.num_snap + j] != done) continue;
        float* dst = p.snap_state + (((size_t)s * p.num_snap + j) * p.hv + vh) * DK * DV;
#pragma unroll
        for (int i = 0; i < DPT; ++i) dst[(size_t)(dg * DPT + i) * DV + c] = S[i];
        if (tid < NCH) {
          __nv_bfloat16* dc = p.snap_conv + (((size_t)s * p.num_snap + j) * p.hv + vh) * 3 * NCH;
          dc[tid] = __float2bfloat16_rn(x0);
          dc[NCH + tid] = __float2bfloat16_rn(x1);
          dc[2 * NCH + tid] = __float2bfloat16_rn(x2);
        }
      }
    }
    __syncthreads();
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
