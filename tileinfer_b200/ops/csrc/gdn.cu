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
// Mapping: one block (decode) or a cluster of blocks (prefill) per (v-head, sequence); thread = (column c of
// the state, quarter dg of the key dimension) with the four quarters of a column in adjacent lanes, so both
// matrix-vector products of a step reduce with two warp shuffles.  A state column never interacts with other
// columns, only the gated norm needs a sum over the head.
//
// Conv history layout: [slot][v-head][3][2*DK + DV]; every v-head keeps its own copy of the q/k
// history of the key head it shares, so blocks never write memory another block reads.
#include <algorithm>

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
  const int* snap_idx;         // [S, NS] index of the snapshot buffer entry of (sequence, point), or nullptr (s * NS + j)
  unsigned* status;            // error bits (a bounded wait that ran out); may be nullptr
};

TI_DEVICE size_t snap_entry(const GdnParams& p, int s, int j) {
  return p.snap_idx != nullptr ? (size_t)p.snap_idx[s * p.num_snap + j] : (size_t)s * p.num_snap + j;
}

template <typename ST> TI_DEVICE float ld_state(const ST* p);
template <> TI_DEVICE float ld_state<float>(const float* p) { return *p; }
template <> TI_DEVICE float ld_state<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename ST> TI_DEVICE void st_state(ST* p, float v);
template <> TI_DEVICE void st_state<float>(float* p, float v) { *p = v; }
template <> TI_DEVICE void st_state<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// Decode form (every sequence of the step has one token): everything of a token in one pass, two block
// barriers.  The tiled kernel below does the same arithmetic per token but stages a tile's worth of q / k / v
// through shared memory, which costs a decode step several microseconds per layer for nothing.
// STAGED (large decode batches): a block walks several sequences of its v-head.  The 64 KB state of the NEXT
// sequence is fetched into shared memory by a bulk copy while the current one is being worked on, and the updated
// state goes back through shared memory with a bulk store, so a block is not idle for a memory round trip per
// sequence (one block per SM fits; with direct loads that was 21 serialised waves at batch 64).
TI_DEVICE void bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
}
TI_DEVICE void bulk_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
TI_DEVICE void bulk_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }

template <int DK, int DV, typename ST, bool STAGED>
__global__ void __launch_bounds__(DV * 4) gdn_token_kernel(const __grid_constant__ GdnParams p, int num_seqs) {
  constexpr int DPT = DK / 4;           // state elements per thread
  constexpr int NCH = 2 * DK + DV;      // conv channels this block needs
  constexpr int NW = DV * 4 / 32;
  constexpr uint32_t kStateBytes = DK * DV * sizeof(ST);
  static_assert(NCH <= DV * 4, "one thread per conv channel");
  __shared__ float qs[DK], ks[DK], vs[DV], red[NW];
  __shared__ __align__(8) unsigned long long full_bar[2];
  extern __shared__ __align__(128) uint8_t stage_raw[];      // STAGED: two state buffers
  ST* sbuf0 = reinterpret_cast<ST*>(stage_raw);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = tid >> 2, dg = tid & 3;
  const int vh = blockIdx.x;
  const int kh = vh / (p.hv / p.hk);
  const int zcol = 2 * p.hk * DK + p.hv * DV + vh * DV;
  const int bcol = 2 * p.hk * DK + 2 * p.hv * DV + vh;
  const int acol = bcol + p.hv;
  const float neg_a = p.neg_a_exp[vh], dtb = p.dt_bias[vh];
  const float nw = p.norm_w[c];
  const float qscale = rsqrtf((float)DK);
  int col = 0;
  float cw0 = 0.f, cw1 = 0.f, cw2 = 0.f, cw3 = 0.f;
  if (tid < NCH) {
    if (tid < DK) col = kh * DK + tid;
    else if (tid < 2 * DK) col = p.hk * DK + kh * DK + (tid - DK);
    else col = 2 * p.hk * DK + vh * DV + (tid - 2 * DK);
    const float4 w = *reinterpret_cast<const float4*>(p.conv_w + (size_t)col * 4);
    cw0 = w.x; cw1 = w.y; cw2 = w.z; cw3 = w.w;
  }
  auto state_ptr = [&](int seq) { return static_cast<ST*>(p.state) + ((size_t)p.slots[seq] * p.hv + vh) * DK * DV; };
  if (STAGED) {
    if (tid == 0) {
      mbar_init(smem_u32(&full_bar[0]), 1);
      mbar_init(smem_u32(&full_bar[1]), 1);
      fence_mbar_init();
      // the recurrent state was last written one step ago: it may be fetched before pdl_wait()
      mbar_expect_tx(smem_u32(&full_bar[0]), kStateBytes);
      bulk_g2s(smem_u32(sbuf0), state_ptr(blockIdx.y), kStateBytes, smem_u32(&full_bar[0]));
    }
    __syncthreads();
  }

  // STAGED also fetches the NEXT sequence's inputs (conv history, projection row entries) one item ahead, so that
  // an item's critical path holds no global round trip.  (STAGED is used for single-token sequences only.)
  struct Inputs { float x0, x1, x2, x3, a, b, z; };
  auto fetch = [&](int seq) {
    Inputs in{0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const int tokn = p.cu ? p.cu[seq] : seq;
    const __nv_bfloat16* rown = p.proj + (size_t)tokn * p.ld;
    const __nv_bfloat16* csn = p.conv_state + ((size_t)p.slots[seq] * p.hv + vh) * 3 * NCH;
    if (tid < NCH) {
      in.x0 = __bfloat162float(csn[tid]);
      in.x1 = __bfloat162float(csn[NCH + tid]);
      in.x2 = __bfloat162float(csn[2 * NCH + tid]);
      in.x3 = __bfloat162float(rown[col]);
    }
    in.a = __bfloat162float(rown[acol]);
    in.b = __bfloat162float(rown[bcol]);
    in.z = __bfloat162float(rown[zcol + c]);
    return in;
  };
  Inputs cur{0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, nxt = cur;

  int k = 0;
  for (int s = blockIdx.y; s < num_seqs; s += gridDim.y, ++k) {
    // cu / slots are written by host copies that precede every kernel of the step; the recurrent state
    // and conv history were last written one step ago: all of this may be read before pdl_wait()
    const int t0 = p.cu ? p.cu[s] : s, t1 = p.cu ? p.cu[s + 1] : s + 1;
    const int slot = p.slots[s];
    ST* Sp = static_cast<ST*>(p.state) + ((size_t)slot * p.hv + vh) * DK * DV;
    ST* sb = sbuf0 + (size_t)(k & 1) * DK * DV;
    if (STAGED && tid == 0 && s + (int)gridDim.y < num_seqs) {
      // next sequence -> the other buffer, once the bulk store that last read that buffer is done with it
      bulk_store_wait_read();
      const uint32_t bar = smem_u32(&full_bar[(k + 1) & 1]);
      mbar_expect_tx(bar, kStateBytes);
      bulk_g2s(smem_u32(sbuf0 + (size_t)((k + 1) & 1) * DK * DV), state_ptr(s + gridDim.y), kStateBytes, bar);
    }
    float S[DPT];
    if (!STAGED) {
#pragma unroll
      for (int i = 0; i < DPT; ++i) S[i] = ld_state<ST>(Sp + (size_t)(dg * DPT + i) * DV + c);
    }
    // conv channel owned by this thread
    __nv_bfloat16* cs = p.conv_state + ((size_t)slot * p.hv + vh) * 3 * NCH;
    float x0 = 0.f, x1 = 0.f, x2 = 0.f;
    if (!STAGED || k == 0) {
      if (tid < NCH) {
        x0 = __bfloat162float(cs[tid]);
        x1 = __bfloat162float(cs[NCH + tid]);
        x2 = __bfloat162float(cs[2 * NCH + tid]);
      }
    }
    if (k == 0) {
      pdl_trigger();
      pdl_wait();                                  // `proj` comes from the preceding projection kernel
    }
    if (STAGED) {
      if (k == 0) {
        cur = fetch(s);
        cur.x0 = x0; cur.x1 = x1; cur.x2 = x2;
      } else {
        cur = nxt;
      }
      x0 = cur.x0; x1 = cur.x1; x2 = cur.x2;
      if (s + (int)gridDim.y < num_seqs) nxt = fetch(s + gridDim.y);
    }
    if (STAGED) {
      // an expired wait is reported in the status word (the state then read is whatever the buffer holds)
      mbar_wait(smem_u32(&full_bar[k & 1]), (uint32_t)((k >> 1) & 1), 2000000000ull, p.status);
#pragma unroll
      for (int i = 0; i < DPT; ++i) S[i] = ld_state<ST>(sb + (size_t)(dg * DPT + i) * DV + c);
    }

    for (int tok = t0; tok < t1; ++tok) {
      const __nv_bfloat16* row = p.proj + (size_t)tok * p.ld;
      if (tid < NCH) {
        const float x3 = STAGED ? cur.x3 : __bfloat162float(row[col]);
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
      const float a = (STAGED ? cur.a : __bfloat162float(row[acol])) + dtb;
      const float sp = a > 20.f ? a : log1pf(__expf(a));
      const float decay = __expf(neg_a * sp);
      const float beta = sigmoid_f(STAGED ? cur.b : __bfloat162float(row[bcol]));

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
        const float z = STAGED ? cur.z : __bfloat162float(row[zcol + c]);
        p.out[(size_t)tok * p.hv * DV + vh * DV + c] = __float2bfloat16_rn(o * rr * nw * silu_f(z));
      }
      if (p.snap_rel != nullptr) {
        const int done = tok - t0 + 1;
        for (int j = 0; j < p.num_snap; ++j) {
          if (p.snap_rel[s * p.num_snap + j] != done) continue;
          float* dst = p.snap_state + (snap_entry(p, s, j) * p.hv + vh) * DK * DV;
#pragma unroll
          for (int i = 0; i < DPT; ++i) dst[(size_t)(dg * DPT + i) * DV + c] = S[i];
          if (tid < NCH) {
            __nv_bfloat16* dc = p.snap_conv + (snap_entry(p, s, j) * p.hv + vh) * 3 * NCH;
            dc[tid] = __float2bfloat16_rn(x0);
            dc[NCH + tid] = __float2bfloat16_rn(x1);
            dc[2 * NCH + tid] = __float2bfloat16_rn(x2);
          }
        }
      }
      __syncthreads();
    }

    if (STAGED) {
#pragma unroll
      for (int i = 0; i < DPT; ++i) st_state<ST>(sb + (size_t)(dg * DPT + i) * DV + c, S[i]);
      fence_proxy_async();                         // generic-proxy writes -> visible to the bulk store
      __syncthreads();
      if (tid == 0) bulk_s2g(Sp, smem_u32(sb), kStateBytes);
    } else {
#pragma unroll
      for (int i = 0; i < DPT; ++i) st_state<ST>(Sp + (size_t)(dg * DPT + i) * DV + c, S[i]);
    }
    if (tid < NCH) {
      cs[tid] = __float2bfloat16_rn(x0);
      cs[NCH + tid] = __float2bfloat16_rn(x1);
      cs[2 * NCH + tid] = __float2bfloat16_rn(x2);
    }
  }
  if (STAGED && tid == 0) bulk_store_wait_all();   // shared memory must outlive the stores that read it
}

// Tokens are processed in tiles of kTT.  Per tile: (1) every conv channel runs its window over the tile's tokens
// (independent global loads, no synchronisation) and the per-token scalars (q/k norms, decay, beta) are worked
// out in parallel; (2) the recurrence walks the tile token by token out of shared memory: two matrix-vector
// products per token, reduced with warp shuffles, nothing else on the serial path; (3) the gated norm and the
// output are again parallel over the tile.  The arithmetic of a token does not depend on the tiling.
constexpr int kTT = 16;

// NS = 1: one block per (v-head, sequence), DV*4 threads.  NS = 4 (prefill): the DV state columns of a head are
// dealt to the NS blocks of a thread-block cluster (columns never interact); the only quantity that spans the
// columns, the sum of squares of the gated norm, is exchanged through distributed shared memory once per tile.
// Both forms add the same four 32-column partial sums in the same order.
TI_DEVICE void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
TI_DEVICE float ld_cluster_f32(const float* local, int rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// Large decode batches: the state columns of a head are dealt to NSPL small blocks (32 columns x DK rows = 16 KB of
// fp32 state each), one block per (sequence, v-head, column part): thousands of independent blocks keep two dozen warps
// per SM in flight, 4 KB of loads each, which streams the recurrent state at HBM speed without any staging (the staged kernel above
// walks ~20 sequences per block one after the other and reaches a third of it).  A warp owns a quarter of the key
// rows and 32 consecutive columns, so every state access is one full 128-byte line; the two matrix-vector
// products meet across the four warps in shared memory.  The gated RMSNorm spans the whole head: this kernel writes
// the un-normalised output and gdn_finish_kernel applies norm * silu(z) in place.  The NSPL blocks of a head form a
// thread-block cluster (they share the q / k conv history).
template <int DK, int DV, typename ST>
__global__ void __launch_bounds__(128, sizeof(ST) == 4 ? 8 : 6) gdn_token_split_kernel(const __grid_constant__ GdnParams p) {
  constexpr int CB = 32, NSPL = DV / CB, DPT = DK / 4;
  constexpr int NCH = 2 * DK + DV, NCHL = 2 * DK + CB;
  constexpr int NCPT = (NCHL + 127) / 128;
  __shared__ float qs[DK], ks[DK], vs[CB], red[2][4], part_s[2][4][CB];
  const int tid = threadIdx.x, lane = tid & 31, dg = tid >> 5;      // warp = quarter of the key rows
  const int c = lane;
  const int part = blockIdx.x % NSPL, vh = blockIdx.x / NSPL, s = blockIdx.y;
  const int kh = vh / (p.hv / p.hk);
  const int slot = p.slots[s];
  const int tok = p.cu ? p.cu[s] : s;
  ST* Sp = static_cast<ST*>(p.state) + ((size_t)slot * p.hv + vh) * DK * DV + part * CB + c;
  float S[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) S[i] = ld_state<ST>(Sp + (size_t)(dg * DPT + i) * DV);     // last written a step ago
  __nv_bfloat16* cs = p.conv_state + ((size_t)slot * p.hv + vh) * 3 * NCH;
  float x0[NCPT], x1[NCPT], x2[NCPT], cw[NCPT][4];
  int col[NCPT], hch[NCPT];
#pragma unroll
  for (int u = 0; u < NCPT; ++u) {
    const int ch = tid + u * 128;
    x0[u] = x1[u] = x2[u] = 0.f;
    col[u] = hch[u] = 0;
    cw[u][0] = cw[u][1] = cw[u][2] = cw[u][3] = 0.f;
    if (ch < NCHL) {
      if (ch < DK) { col[u] = kh * DK + ch; hch[u] = ch; }
      else if (ch < 2 * DK) { col[u] = p.hk * DK + kh * DK + (ch - DK); hch[u] = ch; }
      else { col[u] = 2 * p.hk * DK + vh * DV + part * CB + (ch - 2 * DK); hch[u] = 2 * DK + part * CB + (ch - 2 * DK); }
      const float4 w = *reinterpret_cast<const float4*>(p.conv_w + (size_t)col[u] * 4);
      cw[u][0] = w.x; cw[u][1] = w.y; cw[u][2] = w.z; cw[u][3] = w.w;
      x0[u] = __bfloat162float(cs[hch[u]]);
      x1[u] = __bfloat162float(cs[NCH + hch[u]]);
      x2[u] = __bfloat162float(cs[2 * NCH + hch[u]]);
    }
  }
  const float neg_a = p.neg_a_exp[vh], dtb = p.dt_bias[vh];
  const int bcol = 2 * p.hk * DK + 2 * p.hv * DV + vh, acol = bcol + p.hv;
  pdl_trigger();
  pdl_wait();                                              // `proj` comes from the preceding projection kernel
  const __nv_bfloat16* row = p.proj + (size_t)tok * p.ld;
#pragma unroll
  for (int u = 0; u < NCPT; ++u) {
    const int ch = tid + u * 128;
    if (ch < NCHL) {
      const float x3 = __bfloat162float(row[col[u]]);
      const float y = silu_f(cw[u][0] * x0[u] + cw[u][1] * x1[u] + cw[u][2] * x2[u] + cw[u][3] * x3);
      if (ch < DK) qs[ch] = y;
      else if (ch < 2 * DK) ks[ch - DK] = y;
      else vs[ch - 2 * DK] = y;
      x0[u] = x3;                                          // kept for the history update below
    }
  }
  // The q / k history of a head is read by all NSPL blocks of the cluster and written by part 0: nobody writes
  // before every block of the cluster has read (the blocks of a cluster are co-scheduled).
  cluster_sync_all();
#pragma unroll
  for (int u = 0; u < NCPT; ++u) {
    const int ch = tid + u * 128;
    if (ch < NCHL && (part == 0 || ch >= 2 * DK)) {
      cs[hch[u]] = __float2bfloat16_rn(x1[u]);
      cs[NCH + hch[u]] = __float2bfloat16_rn(x2[u]);
      cs[2 * NCH + hch[u]] = __float2bfloat16_rn(x0[u]);
    }
  }
  __syncthreads();
  float sq = 0.f, sk = 0.f;
  for (int i = tid; i < DK; i += 128) { sq += qs[i] * qs[i]; sk += ks[i] * ks[i]; }
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  if (lane == 0) { red[0][dg] = sq; red[1][dg] = sk; }
  const float a = __bfloat162float(row[acol]) + dtb;
  const float sp = a > 20.f ? a : log1pf(__expf(a));
  const float decay = __expf(neg_a * sp);
  const float beta = sigmoid_f(__bfloat162float(row[bcol]));
  __syncthreads();
  const float qn = rsqrtf(red[0][0] + red[0][1] + red[0][2] + red[0][3] + 1e-6f) * rsqrtf((float)DK);
  const float kn = rsqrtf(red[1][0] + red[1][1] + red[1][2] + red[1][3] + 1e-6f);
  float kv = 0.f;
#pragma unroll
  for (int i = 0; i < DPT; ++i) { S[i] *= decay; kv += S[i] * ks[dg * DPT + i]; }
  part_s[0][dg][c] = kv;
  __syncthreads();
  kv = part_s[0][0][c] + part_s[0][1][c] + part_s[0][2][c] + part_s[0][3][c];
  const float kd = kn * (vs[c] - kv * kn) * beta;
  float o = 0.f;
#pragma unroll
  for (int i = 0; i < DPT; ++i) { S[i] += ks[dg * DPT + i] * kd; o += S[i] * qs[dg * DPT + i]; }
  part_s[1][dg][c] = o;
#pragma unroll
  for (int i = 0; i < DPT; ++i) st_state<ST>(Sp + (size_t)(dg * DPT + i) * DV, S[i]);
  __syncthreads();
  if (dg == 0) {
    o = (part_s[1][0][c] + part_s[1][1][c] + part_s[1][2][c] + part_s[1][3][c]) * qn;
    p.out[(size_t)tok * p.hv * DV + vh * DV + part * CB + c] = __float2bfloat16_rn(o);
  }
}

// gated RMSNorm over the head * silu(z), in place on the un-normalised output of the split kernel: a warp per
// (sequence, v-head)
template <int DK, int DV>
__global__ void __launch_bounds__(256) gdn_finish_kernel(const __grid_constant__ GdnParams p, int num_seqs) {
  constexpr int E = DV / 32;
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();
  if (item >= num_seqs * p.hv) return;
  const int s = item / p.hv, vh = item - s * p.hv;
  const int tok = p.cu ? p.cu[s] : s;
  __nv_bfloat16* o = p.out + (size_t)tok * p.hv * DV + vh * DV + lane * E;
  const __nv_bfloat16* z = p.proj + (size_t)tok * p.ld + 2 * p.hk * DK + p.hv * DV + vh * DV + lane * E;
  float v[E], ss = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    v[e] = __bfloat162float(o[e]);
    ss += v[e] * v[e];
  }
  ss = warp_sum(ss);
  const float rr = rsqrtf(ss / (float)DV + p.eps);
#pragma unroll
  for (int e = 0; e < E; ++e)
    o[e] = __float2bfloat16_rn(v[e] * rr * p.norm_w[lane * E + e] * silu_f(__bfloat162float(z[e])));
}

template <int DK, int DV, typename ST, int NS>
__global__ void __launch_bounds__(DV / NS * 4) gdn_kernel(const __grid_constant__ GdnParams p) {
  constexpr int DPT = DK / 4;           // state elements per thread
  constexpr int CB = DV / NS;           // state columns of this block
  constexpr int NT = CB * 4;            // threads
  constexpr int NCH = 2 * DK + DV;      // conv channels of a head (layout of the conv history)
  constexpr int NCHL = 2 * DK + CB;     // conv channels this block needs: q, k, its own v columns
  constexpr int NCPT = (NCHL + NT - 1) / NT;   // channels per thread
  constexpr int NW = NT / 32;
  constexpr int NG = CB / 32;           // 32-column groups of this block (DV / 32 in total)
  static_assert(CB % 32 == 0 && DV / 32 <= 8, "column groups");
  // q/k rows are padded by 4 floats per quarter so that the four quarters (lanes dg = 0..3 read different
  // quarters at the same time) fall into different banks
  constexpr int DKP = DK + 16;
  __shared__ __align__(16) float qs[kTT][DKP], ks[kTT][DKP], vs[kTT][CB];     // vs holds v, then the un-normalised output
  __shared__ float qn_s[kTT], kn_s[kTT], decay_s[kTT], beta_s[kTT], rr_s[kTT];
  __shared__ float o2_s[2][kTT][NG];    // partial sums of squares per column group (double-buffered by tile)

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = tid >> 2, dg = tid & 3;              // local column, k quarter
  const int part = NS > 1 ? (int)(blockIdx.x % NS) : 0;
  const int vh = blockIdx.x / NS, s = blockIdx.y;
  const int kh = vh / (p.hv / p.hk);
  // cu / slots are written by host copies that precede every kernel of the step; the recurrent state
  // and conv history were last written one step ago: all of this may be read before pdl_wait()
  const int t0 = p.cu ? p.cu[s] : s, t1 = p.cu ? p.cu[s + 1] : s + 1;
  const int slot = p.slots[s];

  ST* Sp = static_cast<ST*>(p.state) + ((size_t)slot * p.hv + vh) * DK * DV + part * CB;
  float2 S2[DPT / 2];                  // S2[i] = state rows (dg*DPT + 2i, 2i+1) of column c
#pragma unroll
  for (int i = 0; i < DPT / 2; ++i) {
    S2[i].x = ld_state<ST>(Sp + (size_t)(dg * DPT + 2 * i) * DV + c);
    S2[i].y = ld_state<ST>(Sp + (size_t)(dg * DPT + 2 * i + 1) * DV + c);
  }

  // conv channels owned by this thread: local channel ch -> index in the head's history, column of `proj`
  __nv_bfloat16* cs = p.conv_state + ((size_t)slot * p.hv + vh) * 3 * NCH;
  float x0[NCPT], x1[NCPT], x2[NCPT], cw[NCPT][4];
  int col[NCPT], hch[NCPT];
#pragma unroll
  for (int u = 0; u < NCPT; ++u) {
    const int ch = tid + u * NT;
    x0[u] = x1[u] = x2[u] = 0.f;
    col[u] = hch[u] = 0;
    cw[u][0] = cw[u][1] = cw[u][2] = cw[u][3] = 0.f;
    if (ch < NCHL) {
      if (ch < DK) { col[u] = kh * DK + ch; hch[u] = ch; }
      else if (ch < 2 * DK) { col[u] = p.hk * DK + kh * DK + (ch - DK); hch[u] = ch; }
      else { col[u] = 2 * p.hk * DK + vh * DV + part * CB + (ch - 2 * DK); hch[u] = 2 * DK + part * CB + (ch - 2 * DK); }
      const float4 w = *reinterpret_cast<const float4*>(p.conv_w + (size_t)col[u] * 4);
      cw[u][0] = w.x; cw[u][1] = w.y; cw[u][2] = w.z; cw[u][3] = w.w;
      x0[u] = __bfloat162float(cs[hch[u]]);
      x1[u] = __bfloat162float(cs[NCH + hch[u]]);
      x2[u] = __bfloat162float(cs[2 * NCH + hch[u]]);
    }
  }
  // q/k history is common to the blocks of a head: block 0 writes it back
  const int zcol = 2 * p.hk * DK + p.hv * DV + vh * DV + part * CB;
  const int bcol = 2 * p.hk * DK + 2 * p.hv * DV + vh;
  const int acol = bcol + p.hv;
  const float neg_a = p.neg_a_exp[vh], dtb = p.dt_bias[vh];
  const float qscale = rsqrtf((float)DK);
  pdl_trigger();
  pdl_wait();                                    // `proj` comes from the preceding projection kernel

  int tile_idx = 0;
  for (int tile0 = t0; tile0 < t1; tile0 += kTT, ++tile_idx) {
    const int nt = min(kTT, t1 - tile0);
    // ---- (1a) conv + SiLU of every channel over the tile.  All global loads of the tile (conv inputs, gate
    //      inputs a / b, output gates z) are issued first, so the tile pays one memory round trip
    constexpr int ZPT = kTT * CB / NT;              // z values per thread
    float zin[ZPT];
#pragma unroll
    for (int k = 0; k < ZPT; ++k) {
      const int e = tid + k * NT, j = e / CB, cc = e - j * CB;
      zin[k] = e < nt * CB ? __bfloat162float(p.proj[(size_t)(tile0 + j) * p.ld + zcol + cc]) : 0.f;
    }
    float a_in = 0.f, b_in = 0.f;
    if (tid < nt) {
      const __nv_bfloat16* row = p.proj + (size_t)(tile0 + tid) * p.ld;
      a_in = __bfloat162float(row[acol]);
      b_in = __bfloat162float(row[bcol]);
    }
    float xin[NCPT][kTT];
#pragma unroll
    for (int u = 0; u < NCPT; ++u)
#pragma unroll
      for (int j = 0; j < kTT; ++j)
        xin[u][j] = (tid + u * NT < NCHL && j < nt) ? __bfloat162float(p.proj[(size_t)(tile0 + j) * p.ld + col[u]]) : 0.f;
#pragma unroll
    for (int u = 0; u < NCPT; ++u) {
      const int ch = tid + u * NT;
      if (ch < NCHL) {
#pragma unroll
        for (int j = 0; j < kTT; ++j) {
          if (j < nt) {
            const float x3 = xin[u][j];
            const float y = silu_f(cw[u][0] * x0[u] + cw[u][1] * x1[u] + cw[u][2] * x2[u] + cw[u][3] * x3);
            x0[u] = x1[u]; x1[u] = x2[u]; x2[u] = x3;
            if (ch < DK) qs[j][ch + 4 * (ch / DPT)] = y;
            else if (ch < 2 * DK) ks[j][(ch - DK) + 4 * ((ch - DK) / DPT)] = y;
            else vs[j][ch - 2 * DK] = y;
            if (p.snap_rel != nullptr && (part == 0 || ch >= 2 * DK)) {   // conv window after token (tile0 + j)
              const int done = tile0 + j - t0 + 1;
              for (int q = 0; q < p.num_snap; ++q) {
                if (p.snap_rel[s * p.num_snap + q] != done) continue;
                __nv_bfloat16* dc = p.snap_conv + (snap_entry(p, s, q) * p.hv + vh) * 3 * NCH;
                dc[hch[u]] = __float2bfloat16_rn(x0[u]);
                dc[NCH + hch[u]] = __float2bfloat16_rn(x1[u]);
                dc[2 * NCH + hch[u]] = __float2bfloat16_rn(x2[u]);
              }
            }
          }
        }
      }
    }
    if (tid < nt) {                                 // gates of token tid
      const float a = a_in + dtb;
      const float sp = a > 20.f ? a : log1pf(__expf(a));
      decay_s[tid] = __expf(neg_a * sp);
      beta_s[tid] = sigmoid_f(b_in);
    }
    __syncthreads();
    // ---- (1b) q / k norms: a warp per token
    for (int j = warp; j < nt; j += NW) {
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
      }
    }
    __syncthreads();
    // ---- (2) the recurrence, token by token, out of shared memory
    for (int j = 0; j < nt; ++j) {
      const float decay = decay_s[j], kn = kn_s[j];
      // 128-bit shared-memory loads and packed fp32 arithmetic (two state elements per instruction); four
      // independent partial sums per product, so no chain of DPT dependent FMAs
      const float4* kj = reinterpret_cast<const float4*>(ks[j] + dg * (DPT + 4));
      const float4* qj = reinterpret_cast<const float4*>(qs[j] + dg * (DPT + 4));
      const float2 dec2 = make_float2(decay, decay);
      float2 kva = make_float2(0.f, 0.f), kvb = kva;
#pragma unroll
      for (int i = 0; i < DPT / 4; ++i) {
        const float4 k4 = kj[i];
        S2[2 * i] = __fmul2_rn(S2[2 * i], dec2);
        S2[2 * i + 1] = __fmul2_rn(S2[2 * i + 1], dec2);
        kva = __ffma2_rn(S2[2 * i], make_float2(k4.x, k4.y), kva);
        kvb = __ffma2_rn(S2[2 * i + 1], make_float2(k4.z, k4.w), kvb);
      }
      float kv = (kva.x + kva.y) + (kvb.x + kvb.y);
      kv += __shfl_xor_sync(0xffffffffu, kv, 1);
      kv += __shfl_xor_sync(0xffffffffu, kv, 2);
      const float delta = (vs[j][c] - kv * kn) * beta_s[j];
      const float kd = kn * delta;
      const float2 kd2 = make_float2(kd, kd);
      float2 oa = make_float2(0.f, 0.f), ob = oa;
#pragma unroll
      for (int i = 0; i < DPT / 4; ++i) {
        const float4 k4 = kj[i], q4 = qj[i];
        S2[2 * i] = __ffma2_rn(make_float2(k4.x, k4.y), kd2, S2[2 * i]);
        S2[2 * i + 1] = __ffma2_rn(make_float2(k4.z, k4.w), kd2, S2[2 * i + 1]);
        oa = __ffma2_rn(S2[2 * i], make_float2(q4.x, q4.y), oa);
        ob = __ffma2_rn(S2[2 * i + 1], make_float2(q4.z, q4.w), ob);
      }
      float o = (oa.x + oa.y) + (ob.x + ob.y);
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      __syncwarp();                                // all four lanes of the column have read vs[j][c]
      if (dg == 0) vs[j][c] = o * qn_s[j];
      if (p.snap_rel != nullptr) {
        const int done = tile0 + j - t0 + 1;
        for (int q = 0; q < p.num_snap; ++q) {
          if (p.snap_rel[s * p.num_snap + q] != done) continue;
          float* dst = p.snap_state + (snap_entry(p, s, q) * p.hv + vh) * DK * DV + part * CB;
#pragma unroll
          for (int i = 0; i < DPT / 2; ++i) {
            dst[(size_t)(dg * DPT + 2 * i) * DV + c] = S2[i].x;
            dst[(size_t)(dg * DPT + 2 * i + 1) * DV + c] = S2[i].y;
          }
        }
      }
    }
    __syncthreads();
    // ---- (3) gated RMSNorm * silu(z): sums of squares per 32-column group (a warp per (token, group)), added in
    //      group order over the whole head (the other blocks' groups come through distributed shared memory)
    float(*o2)[NG] = o2_s[tile_idx & 1];
    for (int e = warp; e < nt * NG; e += NW) {
      const int j = e / NG, gq = e - j * NG;
      const float v = vs[j][gq * 32 + lane];
      const float t = warp_sum(v * v);
      if (lane == 0) o2[j][gq] = t;
    }
    if (NS > 1) cluster_sync_all(); else __syncthreads();
    if (tid < nt) {
      float tot = 0.f;
      for (int r = 0; r < NS; ++r)
        for (int gq = 0; gq < NG; ++gq) tot += (NS > 1 && r != part) ? ld_cluster_f32(&o2[tid][gq], r) : o2[tid][gq];
      rr_s[tid] = rsqrtf(tot / (float)DV + p.eps);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < ZPT; ++k) {
      const int e = tid + k * NT, j = e / CB, cc = e - j * CB;
      if (e < nt * CB)
        p.out[(size_t)(tile0 + j) * p.hv * DV + vh * DV + part * CB + cc] =
            __float2bfloat16_rn(vs[j][cc] * rr_s[j] * p.norm_w[part * CB + cc] * silu_f(zin[k]));
    }
    __syncthreads();                               // the tile buffers are reused
  }

#pragma unroll
  for (int i = 0; i < DPT / 2; ++i) {
    st_state<ST>(Sp + (size_t)(dg * DPT + 2 * i) * DV + c, S2[i].x);
    st_state<ST>(Sp + (size_t)(dg * DPT + 2 * i + 1) * DV + c, S2[i].y);
  }
#pragma unroll
  for (int u = 0; u < NCPT; ++u) {
    const int ch = tid + u * NT;
    if (ch < NCHL && (part == 0 || ch >= 2 * DK)) {
      cs[hch[u]] = __float2bfloat16_rn(x0[u]);
      cs[NCH + hch[u]] = __float2bfloat16_rn(x1[u]);
      cs[2 * NCH + hch[u]] = __float2bfloat16_rn(x2[u]);
    }
  }
  if (NS > 1) cluster_sync_all();                  // nobody leaves while a neighbour may still read its partial sums
}

template <int DK, int DV, typename ST, bool STAGED>
static cudaError_t launch_token(const GdnParams& p, int num_seqs, dim3 grid, cudaStream_t st) {
  auto k = gdn_token_kernel<DK, DV, ST, STAGED>;
  const size_t smem = STAGED ? 2 * (size_t)DK * DV * sizeof(ST) : 0;
  static bool configured = false;
  if (STAGED && !configured) {
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = true;
  }
  return launch_kernel(k, grid, dim3(DV * 4), smem, st, true, p, num_seqs);
}

template <int DK, int DV, typename ST>
static cudaError_t launch_token_split(const GdnParams& p, int num_seqs, cudaStream_t st) {
  constexpr int NSPL = DV / 32;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.hv * NSPL, num_seqs);
  cfg.blockDim = dim3(128);
  cfg.stream = st;
  cudaLaunchAttribute at[2];
  int n = 0;
  if (pdl_enabled()) {
    at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  at[n].id = cudaLaunchAttributeClusterDimension;
  at[n].val.clusterDim.x = NSPL;
  at[n].val.clusterDim.y = 1;
  at[n].val.clusterDim.z = 1;
  ++n;
  cfg.attrs = at;
  cfg.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gdn_token_split_kernel<DK, DV, ST>, p);
  if (e != cudaSuccess) return e;
  return launch_kernel(gdn_finish_kernel<DK, DV>, dim3((num_seqs * p.hv + 7) / 8), dim3(256), 0, st, true, p, num_seqs);
}

// Launch with programmatic stream serialization and, for NS > 1, clusters of NS blocks along x.
template <int DK, int DV, typename ST, int NS>
static cudaError_t launch_gdn(const GdnParams& p, int num_seqs, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.hv * NS, num_seqs);
  cfg.blockDim = dim3(DV / NS * 4);
  cfg.stream = st;
  cudaLaunchAttribute at[2];
  int n = 0;
  if (pdl_enabled()) {
    at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (NS > 1) {
    at[n].id = cudaLaunchAttributeClusterDimension;
    at[n].val.clusterDim.x = NS;
    at[n].val.clusterDim.y = 1;
    at[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = at;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, gdn_kernel<DK, DV, ST, NS>, p);
}

}  // namespace ti

extern "C" {

int ti_gdn_params_size() { return (int)sizeof(ti::GdnParams); }

// state_bf16: 0 = fp32 state pool, 1 = bf16.  (dk, dv) must be (128,128) or (64,64).
// split 1: the columns of a head go to a cluster of 4 (dv 128) or 2 (dv 64) blocks (prefill; measured slower, off
// by default).  split 2: the single-pass kernels for steps in which every sequence has exactly one token (decode):
// one block per (head, sequence) for small batches, column-split blocks for large ones (staged blocks that walk
// several sequences when snapshots are wanted, or with split 3).
int ti_gdn_step(const ti::GdnParams* p, int num_seqs, int dk, int dv, int state_bf16, int split, void* stream) {
  if (num_seqs <= 0) return 0;
  if (p->hv % p->hk) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (split >= 2) {                     // one token per sequence: the single-pass decode kernel
    // more (head, sequence) pairs than two waves of SMs: blocks walk several sequences with staged state
    const bool staged = (long long)p->hv * num_seqs > 2 * 148;
    // large batches without snapshots: column-split blocks (split 3 keeps the staged kernel: tests, comparisons)
    static const long long split_min = [] {
      const char* e = getenv("TI_GDN_SPLIT_MIN");            // (head, sequence) pairs from which the column-split kernel runs
      return e == nullptr ? 2LL * 148 : atoll(e);
    }();
    if ((long long)p->hv * num_seqs > split_min && split == 2 && p->snap_rel == nullptr) {
      if (dk == 128 && dv == 128)
        e = state_bf16 ? ti::launch_token_split<128, 128, __nv_bfloat16>(*p, num_seqs, st) : ti::launch_token_split<128, 128, float>(*p, num_seqs, st);
      else if (dk == 64 && dv == 64)
        e = state_bf16 ? ti::launch_token_split<64, 64, __nv_bfloat16>(*p, num_seqs, st) : ti::launch_token_split<64, 64, float>(*p, num_seqs, st);
      else
        return -3;
      return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
    }
    const int gy = staged ? std::max(1, 148 / p->hv) : num_seqs;
    dim3 grid(p->hv, gy);
    if (dk == 128 && dv == 128) {
      if (staged) e = state_bf16 ? ti::launch_token<128, 128, __nv_bfloat16, true>(*p, num_seqs, grid, st)
                                 : ti::launch_token<128, 128, float, true>(*p, num_seqs, grid, st);
      else e = state_bf16 ? ti::launch_token<128, 128, __nv_bfloat16, false>(*p, num_seqs, grid, st)
                          : ti::launch_token<128, 128, float, false>(*p, num_seqs, grid, st);
    } else if (dk == 64 && dv == 64) {
      if (staged) e = state_bf16 ? ti::launch_token<64, 64, __nv_bfloat16, true>(*p, num_seqs, grid, st)
                                 : ti::launch_token<64, 64, float, true>(*p, num_seqs, grid, st);
      else e = state_bf16 ? ti::launch_token<64, 64, __nv_bfloat16, false>(*p, num_seqs, grid, st)
                          : ti::launch_token<64, 64, float, false>(*p, num_seqs, grid, st);
    } else {
      return -3;
    }
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
  }
  if (dk == 128 && dv == 128) {
    if (split) e = state_bf16 ? ti::launch_gdn<128, 128, __nv_bfloat16, 4>(*p, num_seqs, st) : ti::launch_gdn<128, 128, float, 4>(*p, num_seqs, st);
    else e = state_bf16 ? ti::launch_gdn<128, 128, __nv_bfloat16, 1>(*p, num_seqs, st) : ti::launch_gdn<128, 128, float, 1>(*p, num_seqs, st);
  } else if (dk == 64 && dv == 64) {
    if (split) e = state_bf16 ? ti::launch_gdn<64, 64, __nv_bfloat16, 2>(*p, num_seqs, st) : ti::launch_gdn<64, 64, float, 2>(*p, num_seqs, st);
    else e = state_bf16 ? ti::launch_gdn<64, 64, __nv_bfloat16, 1>(*p, num_seqs, st) : ti::launch_gdn<64, 64, float, 1>(*p, num_seqs, st);
  } else {
    return -3;
  }
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

}  // extern "C"
