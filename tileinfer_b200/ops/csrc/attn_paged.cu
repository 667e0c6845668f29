// GQA attention over a paged KV cache for decode AND variable-length causal prefill, plus the
// kernel that prepares its inputs (per-head RMSNorm(1+w) of q and k, partial RoPE computed from the
// positions, K/V written into their pages).
//
// Replaces kernels/qknorm_rope.py:7-57 (+ the eager norm/RoPE path of model/qwen_36.py:983-1002 and
// the HuggingFace rotary module), kernels/kvcache_store.py:14-71, kernels/gqa_decode_paged.py:37-437
// (one CTA per (sequence, kv group), no split-KV, block-table width fixed at compile time),
// kernels/gqa_varlen.py:34-387 together with the whole-prefix KV gather of
// model/qwen_36.py:1031-1042, and the sigmoid output gate of kernels/act_mul.py.
//
// Cache layout (per layer): K pages [block][kv_head][16 tokens][D], V pages transposed
// [block][kv_head][D][16 tokens].  With V stored token-minor both products read their B operand with
// plain 128/64-bit global loads that cover a page exactly once: no shared-memory staging, no
// ldmatrix.  One warp processes one 16-token page per iteration: S = Q K^T on mma.sync m16n8k16 with
// the (up to 16) query rows = (token, head-of-group) pairs as the A operand, online softmax in the
// exp2 domain in registers, O += P V^T.  Pages are dealt round-robin to the warp streams of a CTA and
// to `nsplit` CTAs (split-KV); a second kernel merges the partial (O, max, sum) triples and applies
// the sigmoid gate.  All sizes (batch, context, block-table width) are run-time values.
#include "common.cuh"

namespace ti {

// ------------------------------------------------------------------------------ q/k prep + KV store
struct QkvPrepParams {
  const __nv_bfloat16* proj;     // [T, ld]: per q head [q(D) | gate(D)], then k heads, then v heads
  const __nv_bfloat16* q_norm;   // [D] (1+w)
  const __nv_bfloat16* k_norm;   // [D]
  const int* positions;          // [T]
  const long long* slot_mapping; // [T] flat slot = block*16 + offset, -1 = do not store
  __nv_bfloat16* q_out;          // [T, hq, D]
  __nv_bfloat16* kcache;         // [blocks, hkv, 16, D]
  __nv_bfloat16* vcache;         // [blocks, hkv, D, 16]
  int ld, hq, hkv, rotary_dim;
  float eps, log2_theta;
  int num_blocks;                // pages in the cache (checked builds verify the slot mapping against it; 0: unknown)
  unsigned* status;              // error bits of the checked build, may be nullptr
};

template <int D>
__global__ void __launch_bounds__(32) qkv_prep_kernel(const __grid_constant__ QkvPrepParams p) {
  constexpr int E = D / 32;                 // elements per lane
  __shared__ float buf[D];
  const int tok = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
  pdl_trigger();
  pdl_wait();
  const __nv_bfloat16* row = p.proj + (size_t)tok * p.ld;
  const bool is_q = head < p.hq, is_k = !is_q && head < p.hq + p.hkv;
  const int kvh = is_q ? 0 : (is_k ? head - p.hq : head - p.hq - p.hkv);
  const __nv_bfloat16* src = is_q ? row + (size_t)head * 2 * D
                                  : row + (size_t)p.hq * 2 * D + (size_t)(is_k ? 0 : p.hkv) * D + (size_t)kvh * D;
  float v[E];
#pragma unroll
  for (int i = 0; i < E; ++i) v[i] = __bfloat162float(src[lane * E + i]);
  const long long slot = p.slot_mapping[tok];
  if (!is_q && !is_k) {                       // V: no norm, no rotation; transposed page
    if (slot < 0) return;
    const long long blk = slot >> 4;
    const int off = (int)(slot & 15);
    if (p.num_blocks > 0 && !TI_CHECK(blk, p.num_blocks, p.status)) return;
    __nv_bfloat16* dst = p.vcache + ((size_t)blk * p.hkv + kvh) * D * 16 + off;
#pragma unroll
    for (int i = 0; i < E; ++i) dst[(size_t)(lane * E + i) * 16] = __float2bfloat16_rn(v[i]);
    return;
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < E; ++i) ss += v[i] * v[i];
  ss = warp_sum(ss);
  const float rr = rsqrtf(ss / (float)D + p.eps);
  const __nv_bfloat16* nw = is_q ? p.q_norm : p.k_norm;
#pragma unroll
  for (int i = 0; i < E; ++i) {
    // the normalised head is rounded to bf16 before the rotation, as the separate norm op would
    buf[lane * E + i] = round_bf16(v[i] * rr * (1.f + __bfloat162float(nw[lane * E + i])));
  }
  __syncwarp();
  const int half = p.rotary_dim >> 1;
  const float pos = (float)p.positions[tok];
  for (int i = lane; i < half; i += 32) {
    const float inv = exp2f(-p.log2_theta * (2.f * (float)i / (float)p.rotary_dim));
    float sn, cs;
    sincosf(pos * inv, &sn, &cs);
    const float x1 = buf[i], x2 = buf[i + half];
    buf[i] = x1 * cs - x2 * sn;
    buf[i + half] = x2 * cs + x1 * sn;
  }
  __syncwarp();
  __nv_bfloat16* dst;
  if (is_q) {
    dst = p.q_out + ((size_t)tok * p.hq + head) * D;
  } else {
    if (slot < 0) return;
    const long long blk = slot >> 4;
    const int off = (int)(slot & 15);
    if (p.num_blocks > 0 && !TI_CHECK(blk, p.num_blocks, p.status)) return;
    dst = p.kcache + (((size_t)blk * p.hkv + kvh) * 16 + off) * D;
  }
#pragma unroll
  for (int i = 0; i < E; ++i) dst[lane * E + i] = __float2bfloat16_rn(buf[lane * E + i]);
}

// ------------------------------------------------------------------------------ attention
struct AttnParams {
  const __nv_bfloat16* q;        // [T, hq, D]
  const __nv_bfloat16* kcache;
  const __nv_bfloat16* vcache;
  const int* block_tables;       // [S, max_blocks]
  const int* positions;          // [T]
  const int* qg_seq;             // [num_qg] sequence of the query group
  const int* qg_tok0;            // [num_qg] first flat token
  const int* qg_ntok;            // [num_qg] tokens in the group (1 or 2; 0 = padding group)
  float* o_part;                 // [num_qg * hkv * nsplit, 16, D]
  float* ml_part;                // [num_qg * hkv * nsplit, 16, 2]
  const __nv_bfloat16* gate_src; // merge: proj [T, ld] (gate of q head h at h*2D + D)
  __nv_bfloat16* out;            // merge: [T, hq*D]
  int hq, hkv, max_blocks, nsplit, ld, num_qg;
  float scale_log2e;
  int num_blocks;                // pages in the cache (checked builds verify block-table entries; 0: unknown)
  unsigned* status;
};

constexpr float kNegBig = -1e30f;

TI_DEVICE uint4 ldg_nc16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
TI_DEVICE uint2 ldg_nc8(const void* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }

struct PageRange { int seq, tok0, ntok, npages, pps; };

TI_DEVICE PageRange page_range(const AttnParams& p, int qg) {
  PageRange r;
  r.ntok = p.qg_ntok[qg];
  r.seq = p.qg_seq[qg];
  r.tok0 = p.qg_tok0[qg];
  const int kvlen = r.ntok > 0 ? p.positions[r.tok0 + r.ntok - 1] + 1 : 0;
  r.npages = (kvlen + 15) >> 4;
  r.pps = max(1, (r.npages + p.nsplit - 1) / p.nsplit);
  return r;
}

template <int D, int DSPLIT>
__global__ void __launch_bounds__(128) attn_kernel(const __grid_constant__ AttnParams p) {
  constexpr int NSTREAM = 4 / DSPLIT;      // page streams per CTA
  constexpr int DH = D / DSPLIT;           // output dims of one warp
  constexpr int NT_O = DH / 8;
  constexpr int NCH = D / 32;              // 16-byte chunks per lane and row in Q K^T
  __shared__ float Osm[NSTREAM][16][D];
  __shared__ float MLsm[NSTREAM][16][2];

  const int qg = blockIdx.x, kh = blockIdx.y, sp = blockIdx.z;
  pdl_trigger();
  pdl_wait();
  const PageRange pr = page_range(p, qg);
  if (pr.ntok == 0) return;
  const int p0 = sp * pr.pps, p1 = min(pr.npages, p0 + pr.pps);
  if (p0 >= p1) return;                    // inactive split: the merge kernel never reads it
  const int G = p.hq / p.hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int stream = warp / DSPLIT, dpart = warp % DSPLIT;

  // rows g and g+8 of the 16-row tile: (token, head of the group)
  int pos[2];
  uint32_t qf[2][NCH][4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + 8 * h;
    const int tk = r / G, hg = r - tk * G;
    const bool valid = tk < pr.ntok;
    pos[h] = valid ? p.positions[pr.tok0 + tk] : -1;
    const __nv_bfloat16* qrow = p.q + ((size_t)(pr.tok0 + (valid ? tk : 0)) * p.hq + kh * G + hg) * D;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const uint4 v = valid ? ldg_nc16(qrow + 8 * (t + 4 * i)) : make_uint4(0, 0, 0, 0);
      qf[h][i][0] = v.x; qf[h][i][1] = v.y; qf[h][i][2] = v.z; qf[h][i][3] = v.w;
    }
  }
  float o[NT_O][4];
#pragma unroll
  for (int n = 0; n < NT_O; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m[2] = {kNegBig, kNegBig}, l[2] = {0.f, 0.f};
  const int tokA = 4 * (g >> 1) + (g & 1);   // page token feeding column g of S tile A; tile B uses tokA + 2

  for (int pg = p0 + stream; pg < p1; pg += NSTREAM) {
    const int blk = p.block_tables[(size_t)pr.seq * p.max_blocks + pg];
    if (p.num_blocks > 0 && !TI_CHECK(blk, p.num_blocks, p.status)) continue;      // checked build: skip a bad page
    const __nv_bfloat16* kbase = p.kcache + ((size_t)blk * p.hkv + kh) * 16 * D;
    float sA[4] = {0.f, 0.f, 0.f, 0.f}, sB[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const uint4 ka = ldg_nc16(kbase + (size_t)tokA * D + 8 * (t + 4 * i));
      const uint4 kb = ldg_nc16(kbase + (size_t)(tokA + 2) * D + 8 * (t + 4 * i));
      mma_bf16_16816(sA, qf[0][i][0], qf[1][i][0], qf[0][i][1], qf[1][i][1], ka.x, ka.y);
      mma_bf16_16816(sA, qf[0][i][2], qf[1][i][2], qf[0][i][3], qf[1][i][3], ka.z, ka.w);
      mma_bf16_16816(sB, qf[0][i][0], qf[1][i][0], qf[0][i][1], qf[1][i][1], kb.x, kb.y);
      mma_bf16_16816(sB, qf[0][i][2], qf[1][i][2], qf[0][i][3], qf[1][i][3], kb.z, kb.w);
    }
    // columns held by this lane: page tokens 4t .. 4t+3  (tile A: 4t, 4t+1; tile B: 4t+2, 4t+3)
    const int j0 = pg * 16 + 4 * t;
    float pv[2][4];
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float sc[4] = {sA[2 * h], sA[2 * h + 1], sB[2 * h], sB[2 * h + 1]};
      float mx = kNegBig;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        sc[e] = (j0 + e <= pos[h]) ? sc[e] * p.scale_log2e : kNegBig;
        mx = fmaxf(mx, sc[e]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float mnew = fmaxf(m[h], mx);
      alpha[h] = exp2f(m[h] - mnew);
      float sum = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pv[h][e] = sc[e] > 0.5f * kNegBig ? exp2f(sc[e] - mnew) : 0.f;
        sum += pv[h][e];
      }
      l[h] = l[h] * alpha[h] + sum;
      m[h] = mnew;
    }
    const uint32_t a0 = pack_bf16(pv[0][0], pv[0][1]), a1 = pack_bf16(pv[1][0], pv[1][1]);
    const uint32_t a2 = pack_bf16(pv[0][2], pv[0][3]), a3 = pack_bf16(pv[1][2], pv[1][3]);
    const __nv_bfloat16* vbase = p.vcache + ((size_t)blk * p.hkv + kh) * D * 16 + (size_t)(dpart * DH) * 16;
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
      const uint2 vv = ldg_nc8(vbase + (size_t)(n * 8 + g) * 16 + 4 * t);
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0]; o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
      mma_bf16_16816(o[n], a0, a1, a2, a3, vv.x, vv.y);
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  // ---- merge the page streams of this CTA
#pragma unroll
  for (int n = 0; n < NT_O; ++n) {
    const int d = dpart * DH + n * 8 + 2 * t;
    Osm[stream][g][d] = o[n][0]; Osm[stream][g][d + 1] = o[n][1];
    Osm[stream][g + 8][d] = o[n][2]; Osm[stream][g + 8][d + 1] = o[n][3];
  }
  if (dpart == 0 && t == 0) {
    MLsm[stream][g][0] = m[0]; MLsm[stream][g][1] = l[0];
    MLsm[stream][g + 8][0] = m[1]; MLsm[stream][g + 8][1] = l[1];
  }
  __syncthreads();
  const size_t item = ((size_t)qg * p.hkv + kh) * p.nsplit + sp;
  for (int idx = tid; idx < 16 * D; idx += 128) {
    const int r = idx / D, d = idx - r * D;
    float M = kNegBig;
#pragma unroll
    for (int s = 0; s < NSTREAM; ++s) M = fmaxf(M, MLsm[s][r][0]);
    float acc = 0.f;
#pragma unroll
    for (int s = 0; s < NSTREAM; ++s) acc += exp2f(MLsm[s][r][0] - M) * Osm[s][r][d];
    p.o_part[(item * 16 + r) * D + d] = acc;
  }
  if (tid < 16) {
    float M = kNegBig, L = 0.f;
#pragma unroll
    for (int s = 0; s < NSTREAM; ++s) M = fmaxf(M, MLsm[s][tid][0]);
#pragma unroll
    for (int s = 0; s < NSTREAM; ++s) L += exp2f(MLsm[s][tid][0] - M) * MLsm[s][tid][1];
    p.ml_part[(item * 16 + tid) * 2] = M;
    p.ml_part[(item * 16 + tid) * 2 + 1] = L;
  }
}

// ---- pipelined variant: K/V pages staged in shared memory by cp.async, a ring per page stream -------------------
// The kernel above issues the loads of a page and waits for them before its MMAs: with few warps per SM the K/V
// stream then runs at a third of the HBM rate for large decode batches.  Here the warps of a stream (one warp, or
// two when the head is split over two warps) prefetch kPipe - 1 pages ahead with cp.async into a ring of shared
// memory; K is stored with its 16-byte chunks XOR-swizzled by the token's parity so that the fragment loads of the
// eight token rows of a quarter warp fall into different banks, V pages are copied as they are.
TI_DEVICE void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
TI_DEVICE void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> TI_DEVICE void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
TI_DEVICE uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
TI_DEVICE uint4 lds128a(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

constexpr int kPipe = 3;       // ring stages per page stream

template <int D, int DSPLIT>
__global__ void __launch_bounds__(128) attn_pipe_kernel(const __grid_constant__ AttnParams p) {
  constexpr int NSTREAM = 4 / DSPLIT;
  constexpr int DH = D / DSPLIT;
  constexpr int NT_O = DH / 8;
  constexpr int NCH = D / 32;
  constexpr int kPage = 16 * D * 2;                     // bytes of a K page (and of a V page)
  constexpr int kStage = 2 * kPage;
  constexpr int TS = 32 * DSPLIT;                       // threads of a stream
  extern __shared__ __align__(128) uint8_t ring_raw[];  // [NSTREAM][kPipe][K page | V page]; reused for the merge
  __shared__ float MLsm[NSTREAM][16][2];

  const int qg = blockIdx.x, kh = blockIdx.y, sp = blockIdx.z;
  pdl_trigger();
  pdl_wait();
  const PageRange pr = page_range(p, qg);
  if (pr.ntok == 0) return;
  const int p0 = sp * pr.pps, p1 = min(pr.npages, p0 + pr.pps);
  if (p0 >= p1) return;
  const int G = p.hq / p.hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int stream = warp / DSPLIT, dpart = warp % DSPLIT;
  const int st_tid = tid - stream * TS;                 // thread index inside the stream

  int pos[2];
  uint32_t qf[2][NCH][4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + 8 * h;
    const int tk = r / G, hg = r - tk * G;
    const bool valid = tk < pr.ntok;
    pos[h] = valid ? p.positions[pr.tok0 + tk] : -1;
    const __nv_bfloat16* qrow = p.q + ((size_t)(pr.tok0 + (valid ? tk : 0)) * p.hq + kh * G + hg) * D;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const uint4 v = valid ? ldg_nc16(qrow + 8 * (t + 4 * i)) : make_uint4(0, 0, 0, 0);
      qf[h][i][0] = v.x; qf[h][i][1] = v.y; qf[h][i][2] = v.z; qf[h][i][3] = v.w;
    }
  }
  float o[NT_O][4];
#pragma unroll
  for (int n = 0; n < NT_O; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m[2] = {kNegBig, kNegBig}, l[2] = {0.f, 0.f};
  const int tokA = 4 * (g >> 1) + (g & 1);

  const uint32_t ring = smem_u32(ring_raw) + (uint32_t)stream * kPipe * kStage;
  const int npg = (p1 - p0 - stream + NSTREAM - 1) / NSTREAM;          // pages of this stream
  // issue the copies of this stream's page number k (K swizzled, V linear) into ring stage k % kPipe
  auto issue = [&](int k) {
    if (k < npg) {
      const int pg = p0 + stream + k * NSTREAM;
      int blk = p.block_tables[(size_t)pr.seq * p.max_blocks + pg];
      if (p.num_blocks > 0 && !TI_CHECK(blk, p.num_blocks, p.status)) blk = 0;    // checked build: never leave the cache
      const uint8_t* kg = reinterpret_cast<const uint8_t*>(p.kcache + ((size_t)blk * p.hkv + kh) * 16 * D);
      const uint8_t* vg = reinterpret_cast<const uint8_t*>(p.vcache + ((size_t)blk * p.hkv + kh) * D * 16);
      const uint32_t ks = ring + (uint32_t)(k % kPipe) * kStage, vs = ks + kPage;
      constexpr int kChunks = kPage / 16, kRowChunks = D * 2 / 16;     // 16-byte chunks per page / per token row
#pragma unroll
      for (int c = st_tid; c < kChunks; c += TS) {
        const int tok = c / kRowChunks, cc = c - tok * kRowChunks;
        cp_async16(ks + (uint32_t)(tok * kRowChunks + (cc ^ ((tok & 1) << 2))) * 16u, kg + (size_t)c * 16);
        cp_async16(vs + (uint32_t)c * 16u, vg + (size_t)c * 16);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int k = 0; k < kPipe - 1; ++k) issue(k);

  for (int k = 0; k < npg; ++k) {
    cp_async_wait<kPipe - 2>();
    if (DSPLIT == 1) __syncwarp();
    else asm volatile("bar.sync %0, %1;\n" ::"r"(1 + stream), "r"(TS) : "memory");
    issue(k + kPipe - 1);                                // refills the stage consumed in the previous iteration
    const int pg = p0 + stream + k * NSTREAM;
    const uint32_t ks = ring + (uint32_t)(k % kPipe) * kStage, vs = ks + kPage;
    constexpr int kRowChunks = D * 2 / 16;
    float sA[4] = {0.f, 0.f, 0.f, 0.f}, sB[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t rowA = ks + (uint32_t)(tokA * kRowChunks) * 16u, rowB = ks + (uint32_t)((tokA + 2) * kRowChunks) * 16u;
    const int swz = (tokA & 1) << 2;                     // tokA + 2 has the same parity
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const uint4 ka = lds128a(rowA + (uint32_t)((t + 4 * i) ^ swz) * 16u);
      const uint4 kb = lds128a(rowB + (uint32_t)((t + 4 * i) ^ swz) * 16u);
      mma_bf16_16816(sA, qf[0][i][0], qf[1][i][0], qf[0][i][1], qf[1][i][1], ka.x, ka.y);
      mma_bf16_16816(sA, qf[0][i][2], qf[1][i][2], qf[0][i][3], qf[1][i][3], ka.z, ka.w);
      mma_bf16_16816(sB, qf[0][i][0], qf[1][i][0], qf[0][i][1], qf[1][i][1], kb.x, kb.y);
      mma_bf16_16816(sB, qf[0][i][2], qf[1][i][2], qf[0][i][3], qf[1][i][3], kb.z, kb.w);
    }
    const int j0 = pg * 16 + 4 * t;
    float pv[2][4];
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float sc[4] = {sA[2 * h], sA[2 * h + 1], sB[2 * h], sB[2 * h + 1]};
      float mx = kNegBig;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        sc[e] = (j0 + e <= pos[h]) ? sc[e] * p.scale_log2e : kNegBig;
        mx = fmaxf(mx, sc[e]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float mnew = fmaxf(m[h], mx);
      alpha[h] = exp2f(m[h] - mnew);
      float sum = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pv[h][e] = sc[e] > 0.5f * kNegBig ? exp2f(sc[e] - mnew) : 0.f;
        sum += pv[h][e];
      }
      l[h] = l[h] * alpha[h] + sum;
      m[h] = mnew;
    }
    const uint32_t a0 = pack_bf16(pv[0][0], pv[0][1]), a1 = pack_bf16(pv[1][0], pv[1][1]);
    const uint32_t a2 = pack_bf16(pv[0][2], pv[0][3]), a3 = pack_bf16(pv[1][2], pv[1][3]);
    const uint32_t vrow = vs + (uint32_t)(dpart * DH) * 32u + (uint32_t)g * 32u + (uint32_t)t * 8u;
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
      const uint2 vv = lds64(vrow + (uint32_t)n * 256u);
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0]; o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
      mma_bf16_16816(o[n], a0, a1, a2, a3, vv.x, vv.y);
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  __syncthreads();                                       // every stream is done with its ring: reuse it for the merge
  float(*Osm)[16][D] = reinterpret_cast<float(*)[16][D]>(ring_raw);
#pragma unroll
  for (int n = 0; n < NT_O; ++n) {
    const int d = dpart * DH + n * 8 + 2 * t;
    Osm[stream][g][d] = o[n][0]; Osm[stream][g][d + 1] = o[n][1];
    Osm[stream][g + 8][d] = o[n][2]; Osm[stream][g + 8][d + 1] = o[n][3];
  }
  if (dpart == 0 && t == 0) {
    MLsm[stream][g][0] = m[0]; MLsm[stream][g][1] = l[0];
    MLsm[stream][g + 8][0] = m[1]; MLsm[stream][g + 8][1] = l[1];
  }
  __syncthreads();
  const size_t item = ((size_t)qg * p.hkv + kh) * p.nsplit + sp;
  for (int idx = tid; idx < 16 * D; idx += 128) {
    const int r = idx / D, d = idx - r * D;
    float M = kNegBig;
#pragma unroll
    for (int s = 0; s < NSTREAM; ++s) M = fmaxf(M, MLsm[s][r][0]);
    float acc = 0.f;
#pragma unroll
    for (int s = 0; s < NSTREAM; ++s) acc += exp2f(MLsm[s][r][0] - M) * Osm[s][r][d];
    p.o_part[(item * 16 + r) * D + d] = acc;
  }
  if (tid < 16) {
    float M = kNegBig, L = 0.f;
#pragma unroll
    for (int s = 0; s < NSTREAM; ++s) M = fmaxf(M, MLsm[s][tid][0]);
#pragma unroll
    for (int s = 0; s < NSTREAM; ++s) L += exp2f(MLsm[s][tid][0] - M) * MLsm[s][tid][1];
    p.ml_part[(item * 16 + tid) * 2] = M;
    p.ml_part[(item * 16 + tid) * 2 + 1] = L;
  }
}

// Combines the split-KV partials of one (query group, kv head, row), normalises, applies the sigmoid
// output gate and writes bf16 [T, hq*D].  One block per row: the split weights are worked out once in
// shared memory, then every thread owns two adjacent output dims and sums the partials with independent
// (unrolled) loads, so the kernel costs a few dependent memory round trips whatever the split count.
constexpr int kMaxSplit = 64;
template <int D>
__global__ void __launch_bounds__(D / 2) attn_merge_kernel(const __grid_constant__ AttnParams p) {
  __shared__ float w_s[kMaxSplit], wl_s[kMaxSplit];
  const int qg = blockIdx.x, kh = blockIdx.y, r = blockIdx.z, tid = threadIdx.x;
  pdl_trigger();
  pdl_wait();
  const PageRange pr = page_range(p, qg);
  const int G = p.hq / p.hkv;
  if (pr.ntok == 0 || r >= pr.ntok * G) return;
  const int nact = (pr.npages + pr.pps - 1) / pr.pps;
  const size_t item0 = ((size_t)qg * p.hkv + kh) * p.nsplit;
  for (int s = tid; s < nact; s += D / 2) {
    const float2 ml = *reinterpret_cast<const float2*>(p.ml_part + ((item0 + s) * 16 + r) * 2);
    w_s[s] = ml.x;
    wl_s[s] = ml.y;
  }
  __syncthreads();
  float M = kNegBig;
  for (int s = 0; s < nact; ++s) M = fmaxf(M, w_s[s]);
  __syncthreads();
  for (int s = tid; s < nact; s += D / 2) {
    const float w = exp2f(w_s[s] - M);
    w_s[s] = w;
    wl_s[s] *= w;
  }
  __syncthreads();
  const int d = tid * 2;
  float a0 = 0.f, a1 = 0.f, L = 0.f;
  const float* src = p.o_part + (item0 * 16 + r) * D + d;
#pragma unroll 8
  for (int s = 0; s < nact; ++s) {
    const float2 o = *reinterpret_cast<const float2*>(src + (size_t)s * 16 * D);
    a0 += w_s[s] * o.x;
    a1 += w_s[s] * o.y;
    L += wl_s[s];
  }
  const int tk = r / G, hg = r - tk * G;
  const int tok = pr.tok0 + tk, head = kh * G + hg;
  const uint32_t gw = *reinterpret_cast<const uint32_t*>(p.gate_src + (size_t)tok * p.ld + (size_t)head * 2 * D + D + d);
  const float inv = 1.f / L;
  *reinterpret_cast<uint32_t*>(p.out + (size_t)tok * p.hq * D + (size_t)head * D + d) =
      pack_bf16(a0 * inv * sigmoid_f(bf16lo(gw)), a1 * inv * sigmoid_f(bf16hi(gw)));
}

}  // namespace ti

template <int D, int DSPLIT>
static void launch_attn_pipe(const ti::AttnParams& p, dim3 grid, cudaStream_t st) {
  constexpr size_t smem = (size_t)(4 / DSPLIT) * ti::kPipe * 2 * 16 * D * 2;
  static bool configured = false;
  auto k = ti::attn_pipe_kernel<D, DSPLIT>;
  if (!configured) {
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = true;
  }
  ti::launch_kernel(k, grid, dim3(128), smem, st, true, p);
}

extern "C" {

int ti_qkv_prep_params_size() { return (int)sizeof(ti::QkvPrepParams); }
int ti_attn_params_size() { return (int)sizeof(ti::AttnParams); }

int ti_qkv_prep(const ti::QkvPrepParams* p, int T, int D, void* stream) {
  if (T <= 0) return 0;
  dim3 grid(T, p->hq + 2 * p->hkv);
  cudaStream_t st = (cudaStream_t)stream;
  if (p->rotary_dim > D || (p->rotary_dim & 1)) return -2;
  if (D == 256) ti::launch_kernel(ti::qkv_prep_kernel<256>, grid, dim3(32), 0, st, true, *p);
  else if (D == 128) ti::launch_kernel(ti::qkv_prep_kernel<128>, grid, dim3(32), 0, st, true, *p);
  else if (D == 64) ti::launch_kernel(ti::qkv_prep_kernel<64>, grid, dim3(32), 0, st, true, *p);
  else return -3;
  return (int)cudaGetLastError();
}

// Launches the split-KV attention kernel and the merge/gate kernel.  The cp.async-pipelined kernel is the default
// (measured faster from batch 1 / 256 tokens of context to batch 64 / 8192); TI_ATTN_PIPE=0 selects the direct-load
// kernel.
int ti_attn_paged(const ti::AttnParams* p, int D, void* stream) {
  if (p->num_qg <= 0) return 0;
  const int G = p->hq / p->hkv;
  if (p->hq % p->hkv || G > 16 || p->nsplit < 1 || p->nsplit > ti::kMaxSplit) return -2;
  dim3 grid(p->num_qg, p->hkv, p->nsplit), mgrid(p->num_qg, p->hkv, 16);
  cudaStream_t st = (cudaStream_t)stream;
  static const int pipe_mode = [] {
    const char* e = getenv("TI_ATTN_PIPE");
    return e == nullptr ? -1 : atoi(e);
  }();
  const bool pipe = pipe_mode != 0;
  if (pipe) {
    if (D == 256) {
      launch_attn_pipe<256, 2>(*p, grid, st);
      ti::launch_kernel(ti::attn_merge_kernel<256>, mgrid, dim3(128), 0, st, true, *p);
    } else if (D == 128) {
      launch_attn_pipe<128, 1>(*p, grid, st);
      ti::launch_kernel(ti::attn_merge_kernel<128>, mgrid, dim3(64), 0, st, true, *p);
    } else if (D == 64) {
      launch_attn_pipe<64, 1>(*p, grid, st);
      ti::launch_kernel(ti::attn_merge_kernel<64>, mgrid, dim3(32), 0, st, true, *p);
    } else {
      return -3;
    }
    return (int)cudaGetLastError();
  }
  if (D == 256) {
    ti::launch_kernel(ti::attn_kernel<256, 2>, grid, dim3(128), 0, st, true, *p);
    ti::launch_kernel(ti::attn_merge_kernel<256>, mgrid, dim3(128), 0, st, true, *p);
  } else if (D == 128) {
    ti::launch_kernel(ti::attn_kernel<128, 1>, grid, dim3(128), 0, st, true, *p);
    ti::launch_kernel(ti::attn_merge_kernel<128>, mgrid, dim3(64), 0, st, true, *p);
  } else if (D == 64) {
    ti::launch_kernel(ti::attn_kernel<64, 1>, grid, dim3(128), 0, st, true, *p);
    ti::launch_kernel(ti::attn_merge_kernel<64>, mgrid, dim3(32), 0, st, true, *p);
  } else {
    return -3;
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
