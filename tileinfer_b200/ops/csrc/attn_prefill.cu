// Variable-length causal GQA attention for prefill chunks on the 5th-generation tensor cores.
//
// Replaces the reference's warp-specialised prefill kernel (kernels/gqa_varlen.py:187-362, mma.sync tiles fed by
// plain loads, shapes fixed at JIT time) together with the gather of the whole cached prefix into a dense K/V
// copy before every later chunk (model/qwen_36.py:1031-1042).  Here a CTA owns 128 query tokens of one head and
// walks the sequence's KV pages in tiles of 128 keys straight out of the paged cache:
//
//   warp 0  TMA producer: Q tile once (4 swizzled 64-column slabs), then per KV tile 8 K pages, each ONE 4-D copy
//           ([16 tokens][D] in the cache -> [2 groups of 8 keys][D/64 slabs][8][64], 128-byte swizzle);
//   warp 6  TMA producer of the 8 V pages per tile ([D][16 tokens] as stored: each page is exactly the B operand
//           of one k = 16 step of P V, 32-byte swizzle); pages are addressed through the block table;
//   warp 1  MMA issuer: S = Q K^T (tcgen05.mma kind::f16, M = N = 128, accumulator in TMEM, two S buffers so the
//           next tile's S is computed while the softmax works on this one), then O += P V (N = D);
//   warps 2-5  softmax: one thread per query row (= TMEM lane): scale, causal mask, running maximum in the exp2
//           domain with lazy rescaling (O in TMEM is only touched when the maximum grew by more than 2^8),
//           P written to shared memory as the bf16 A operand of the second product; at the end O / l times the
//           sigmoid output gate goes to [T, hq*D].
//
// TMEM: S0 | S1 | O = 128 + 128 + D columns (512 allocated).  Shared memory at D = 256: Q 64 KB, K 64 KB,
// V 64 KB, P 32 KB.  Causal alignment is by absolute position (bottom-right): a chunk that continues a cached
// prefix sees all of it.  Every wait is bounded; on expiry the status word is set, all roles leave their loops
// and TMEM is freed.  No load carries a cluster-multicast qualifier.
#include <map>
#include <mutex>
#include <tuple>

#include "tcgen05.cuh"

namespace ti {

struct AttnPrefillParams {
  alignas(64) CUtensorMap map_q;   // bf16 [T][hq*D], box {64, 128}, 128B swizzle
  alignas(64) CUtensorMap map_k;   // bf16 [blocks*hkv*2 groups][D/64 slabs][8 keys][64], box {64, 8, D/64, 2}, 128B swizzle
  alignas(64) CUtensorMap map_v;   // bf16 [blocks*hkv*D][16], box {16, D}, 32B swizzle
  const int* block_tables;         // [S, max_blocks]
  const int* positions;            // [T]
  const int* qt_seq;               // [num_tiles] sequence of the query tile
  const int* qt_tok0;              // [num_tiles] first flat token
  const int* qt_ntok;              // [num_tiles] tokens in the tile (1..128; 0 = padding tile)
  const __nv_bfloat16* gate_src;   // proj [T, ld]: gate of q head h at h*2D + D
  __nv_bfloat16* out;              // [T, hq*D]
  unsigned* status;
  int hq, hkv, max_blocks, ld;
  float scale_log2e;
};

constexpr unsigned long long kAttnWaitNs = 500000000ull;
constexpr int kAttnThreads = 224;        // warp 0: Q/K producer, 1: MMA issuer, 2..5: softmax, 6: V producer
constexpr int kAttnProducerV = 6;
constexpr float kMaskVal = -1e30f;
constexpr float kRescaleGap = 8.f;       // log2 units the running maximum may lag behind before O is rescaled

template <int D> struct AttnPrefillGeom {
  static constexpr int kSlabs = D / 64;
  static constexpr int kQBytes = kSlabs * 128 * 128;
  static constexpr int kKBytes = kSlabs * 128 * 128;
  static constexpr int kVPage = D * 32;
  static constexpr int kVBytes = 8 * kVPage;
  static constexpr int kPBytes = 2 * 128 * 128;
  static constexpr int kBarBytes = 128;
  static constexpr size_t kNeeded = (size_t)kQBytes + kKBytes + kVBytes + kPBytes + kBarBytes + 1024;
  // one CTA per SM (the kernel takes all 512 TMEM columns)
  static constexpr size_t kSmem = kNeeded > 120 * 1024 ? kNeeded : 120 * 1024;
};

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1) attn_prefill_kernel(const __grid_constant__ AttnPrefillParams p) {
  using G = AttnPrefillGeom<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t q_s = smem_u32(smem), k_s = q_s + G::kQBytes, v_s = k_s + G::kKBytes, p_s = v_s + G::kVBytes;
  const uint32_t bars = p_s + G::kPBytes;
  const uint32_t q_full = bars, k_full = bars + 8, k_empty = bars + 16, v_full = bars + 24, v_empty = bars + 32,
                 s_full0 = bars + 40, p_full = bars + 56, p_empty = bars + 64, tmem_slot = bars + 72;
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem + G::kQBytes + G::kKBytes + G::kVBytes + G::kPBytes + 72);
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, head = blockIdx.y;
  const int ntok = p.qt_ntok[tile];
  if (ntok <= 0) return;                                   // padding tile (uniform over the CTA)
  const int seq = p.qt_seq[tile], tok0 = p.qt_tok0[tile];
  const int kh = head / (p.hq / p.hkv);
  const int kv_len = p.positions[tok0 + ntok - 1] + 1;
  const int npages = (kv_len + 15) >> 4;
  const int ntiles = (kv_len + 127) >> 7;

  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full0, 1);
    mbar_init(s_full0 + 8, 1);
    mbar_init(p_full, 128);
    mbar_init(p_empty, 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  volatile int* abort_flag = &s_abort;

  if (warp == 0 || warp == kAttnProducerV) {
    // ------------------------------------------------------------ TMA producers: warp 0 Q and K, warp 6 V
    // (one thread's wait / expect / copy sequence is slower than the tensor pipe consumes a tile, so K and V are
    // requested by two threads; a K page is ONE 4-D copy: [2 groups of 8 keys][kSlabs][8][64 columns])
    if (elect_one()) {
      const int* bt = p.block_tables + (size_t)seq * p.max_blocks;
      if (warp == 0) {
        mbar_expect_tx(q_full, G::kQBytes);
#pragma unroll
        for (int s = 0; s < G::kSlabs; ++s) tma_load_2d(q_s + s * (128 * 128), &p.map_q, head * D + s * 64, tok0, q_full);
        for (int j = 0; j < ntiles && !*abort_flag; ++j) {
          int blk[8];
#pragma unroll
          for (int g = 0; g < 8; ++g) blk[g] = bt[min(j * 8 + g, npages - 1)];   // pages past the end repeat the last one (masked)
          if (j > 0 && !mbar_wait(k_empty, (uint32_t)((j - 1) & 1), kAttnWaitNs, p.status)) { *abort_flag = 1; break; }
          mbar_expect_tx(k_full, G::kKBytes);
#pragma unroll
          for (int g = 0; g < 8; ++g)
            tma_load_4d(k_s + g * (G::kSlabs * 2048), &p.map_k, 0, 0, 0, (blk[g] * p.hkv + kh) * 2, k_full);
        }
      } else {
        for (int j = 0; j < ntiles && !*abort_flag; ++j) {
          int blk[8];
#pragma unroll
          for (int g = 0; g < 8; ++g) blk[g] = bt[min(j * 8 + g, npages - 1)];
          if (j > 0 && !mbar_wait(v_empty, (uint32_t)((j - 1) & 1), kAttnWaitNs, p.status)) { *abort_flag = 1; break; }
          mbar_expect_tx(v_full, G::kVBytes);
#pragma unroll
          for (int g = 0; g < 8; ++g) tma_load_2d(v_s + g * G::kVPage, &p.map_v, 0, (blk[g] * p.hkv + kh) * D, v_full);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = idesc_f16_bf16(128, 128), idesc_o = idesc_f16_bf16(128, D);
      auto issue_qk = [&](int j) {
        const uint32_t d = tmem_base + (uint32_t)(j & 1) * 128u;
#pragma unroll
        for (int s = 0; s < G::kSlabs; ++s)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)                     // K: per 8-key group the kSlabs 64-column slabs side by side
            umma_bf16(d, smem_desc_sw128(q_s + s * (128 * 128) + ks * 32),
                      smem_desc_sw128_sbo(k_s + s * 1024 + ks * 32, G::kSlabs * 1024), idesc_s, (s | ks) ? 1u : 0u);
        umma_commit(k_empty);
        umma_commit(s_full0 + 8 * (j & 1));
      };
      bool ok = mbar_wait(q_full, 0, kAttnWaitNs, p.status) && mbar_wait(k_full, 0, kAttnWaitNs, p.status);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; j < ntiles && ok && !*abort_flag; ++j) {
        if (j + 1 < ntiles) {
          ok = mbar_wait(k_full, (uint32_t)((j + 1) & 1), kAttnWaitNs, p.status);
          if (!ok) break;
          tc_fence_after();
          issue_qk(j + 1);
        }
        ok = mbar_wait(p_full, (uint32_t)(j & 1), kAttnWaitNs, p.status) && mbar_wait(v_full, (uint32_t)(j & 1), kAttnWaitNs, p.status);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int g = 0; g < 8; ++g)
          umma_bf16(tmem_base + 256u, smem_desc_sw128(p_s + (g >> 2) * (128 * 128) + (g & 3) * 32),
                    smem_desc_sw32(v_s + g * G::kVPage), idesc_o, (j | g) ? 1u : 0u);
        umma_commit(v_empty);
        umma_commit(p_empty);
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue: thread = query row
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const bool valid = r < ntok;
    const int pos = p.positions[tok0 + (valid ? r : ntok - 1)];
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    float m_used = kMaskVal, l = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      ok = ok && !*abort_flag && mbar_wait(s_full0 + 8 * (j & 1), (uint32_t)((j >> 1) & 1), kAttnWaitNs, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_addr = lane_base + (uint32_t)(j & 1) * 128u;
      const int key0 = j * 128;
      const bool need_mask = key0 + 127 > pos;
      // ---- pass 1: row maximum
      float mx = kMaskVal;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(s_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(v[i]) * p.scale_log2e;
          if (need_mask && key0 + c * 32 + i > pos) s = kMaskVal;
          mx = fmaxf(mx, s);
        }
      }
      const float m_new = fmaxf(m_used, mx);
      const bool resc = m_new - m_used > kRescaleGap;
      float alpha = 1.f;
      if (resc) {
        alpha = exp2f(m_used - m_new);
        l *= alpha;
        m_used = m_new;
      }
      // ---- P buffer free and O quiescent: the previous tile's P V has completed
      if (j > 0) {
        ok = mbar_wait(p_empty, (uint32_t)((j - 1) & 1), kAttnWaitNs, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, resc)) {
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[32];
            tmem_ld32(lane_base + 256u + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st32(lane_base + 256u + c * 32, v);
          }
          tmem_st_wait();
        }
      }
      // ---- pass 2: P = exp2(S - m), row sum, bf16 A operand in the 128-byte-swizzled K-major layout
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(s_addr + c * 32, v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float s0 = __uint_as_float(v[i]) * p.scale_log2e, s1 = __uint_as_float(v[i + 1]) * p.scale_log2e;
          if (need_mask) {
            if (key0 + c * 32 + i > pos) s0 = kMaskVal;
            if (key0 + c * 32 + i + 1 > pos) s1 = kMaskVal;
          }
          const float p0 = exp2f(s0 - m_used), p1 = exp2f(s1 - m_used);
          sum += p0 + p1;
          pk[i >> 1] = pack_bf16(p0, p1);
        }
        const uint32_t row_addr = p_s + (uint32_t)(c >> 1) * (128 * 128) + (uint32_t)r * 128u;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t chunk = (uint32_t)((c & 1) * 4 + q4) ^ (uint32_t)(r & 7);
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(row_addr + chunk * 16u), "r"(pk[4 * q4]),
                       "r"(pk[4 * q4 + 1]), "r"(pk[4 * q4 + 2]), "r"(pk[4 * q4 + 3])
                       : "memory");
        }
      }
      l += sum;
      tc_fence_before();
      fence_proxy_async();
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(p_full) : "memory");
    }
    // ---- epilogue: O / l * sigmoid(gate) -> bf16
    if (ok) {
      ok = mbar_wait(p_empty, (uint32_t)((ntiles - 1) & 1), kAttnWaitNs, p.status);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l;
      const size_t tok = (size_t)tok0 + (valid ? r : 0);
      const __nv_bfloat16* gate = p.gate_src + tok * p.ld + (size_t)head * 2 * D + D;
      __nv_bfloat16* dst = p.out + tok * ((size_t)p.hq * D) + (size_t)head * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(lane_base + 256u + c * 32, v);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const uint4 gw = *reinterpret_cast<const uint4*>(gate + c * 32 + q4 * 8);
            const uint32_t g4[4] = {gw.x, gw.y, gw.z, gw.w};
            uint32_t o4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              o4[e] = pack_bf16(__uint_as_float(v[q4 * 8 + 2 * e]) * inv * sigmoid_f(bf16lo(g4[e])),
                                __uint_as_float(v[q4 * 8 + 2 * e + 1]) * inv * sigmoid_f(bf16hi(g4[e])));
            *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
          }
        }
      }
    } else {
      *abort_flag = 1;
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

struct AMapKey {
  const void* base;
  long long d0, d1;
  int b0, b1, swz;
  bool operator<(const AMapKey& o) const {
    return std::tie(base, d0, d1, b0, b1, swz) < std::tie(o.base, o.d0, o.d1, o.b0, o.b1, o.swz);
  }
};

// bf16 2-D tensor map [d1 rows][d0 columns] with row pitch d0 elements, box {b0, b1}; cached (an encode is a driver call)
static int bf16_map_2d(CUtensorMap* dst, const void* base, long long d0, long long d1, int b0, int b1, CUtensorMapSwizzle swz) {
  static std::map<AMapKey, CUtensorMap> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const AMapKey key{base, d0, d1, b0, b1, (int)swz};
  auto it = cache.find(key);
  if (it == cache.end()) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return 999;
    CUtensorMap m;
    const cuuint64_t dims[2] = {(cuuint64_t)d0, (cuuint64_t)d1};
    const cuuint64_t strides[1] = {(cuuint64_t)d0 * 2};
    const cuuint32_t box[2] = {(cuuint32_t)b0, (cuuint32_t)b1};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1000 + (int)r;
    if (cache.size() > 4096) cache.clear();
    it = cache.emplace(key, m).first;
  }
  *dst = it->second;
  return 0;
}

// K cache [rows = blocks*hkv*16][D] seen as [groups of 8 rows][D/64 slabs][8 rows][64 columns]: one copy brings a
// 16-key page as two 8-key groups with their column slabs side by side (the layout the QK^T descriptors walk).
static int bf16_map_kpage(CUtensorMap* dst, const void* base, int D, long long rows) {
  static std::map<AMapKey, CUtensorMap> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const AMapKey key{base, D, rows, 64, 8, -1};
  auto it = cache.find(key);
  if (it == cache.end()) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return 999;
    CUtensorMap m;
    const cuuint64_t dims[4] = {64, 8, (cuuint64_t)(D / 64), (cuuint64_t)(rows / 8)};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 2, 128, (cuuint64_t)D * 16};
    const cuuint32_t box[4] = {64, 8, (cuuint32_t)(D / 64), 2};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1000 + (int)r;
    if (cache.size() > 4096) cache.clear();
    it = cache.emplace(key, m).first;
  }
  *dst = it->second;
  return 0;
}

template <int D>
static int launch_attn_prefill(const AttnPrefillParams& p, int num_tiles, cudaStream_t st) {
  static bool configured = false;
  auto k = attn_prefill_kernel<D>;
  if (!configured) {
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AttnPrefillGeom<D>::kSmem);
    configured = true;
  }
  k<<<dim3(num_tiles, p.hq), kAttnThreads, AttnPrefillGeom<D>::kSmem, st>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace ti

extern "C" {

// out[tok, head*D + d] = softmax(q k^T / sqrt(D), causal by position) v * sigmoid(gate) for the tokens of the listed
// query tiles (up to 128 consecutive tokens of one sequence each; longest first gives the best balance).
// q: bf16 [T, hq, D] (normalised, rotated); kcache / vcache: the paged cache of this layer, `num_blocks` pages;
// positions: absolute position of every flat token; gate_src: the projection rows [T, ld] holding the gates.
int ti_attn_prefill(const void* q, int T, const void* kcache, const void* vcache, int num_blocks, const void* block_tables,
                    const void* positions, const void* qt_seq, const void* qt_tok0, const void* qt_ntok, int num_tiles,
                    const void* gate_src, void* out, int hq, int hkv, int max_blocks, int ld, float scale_log2e, int D,
                    void* status, void* stream) {
  if (num_tiles <= 0) return 0;
  if (hq % hkv || (D != 64 && D != 128 && D != 256) || T < 1 || num_blocks < 1) return -2;
  // the gate and the output are read / written 16 bytes at a time: refuse layouts that would make those accesses misaligned
  if ((ld & 7) || (reinterpret_cast<uintptr_t>(gate_src) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return -4;
  ti::AttnPrefillParams p = {};
  int rc = ti::bf16_map_2d(&p.map_q, q, (long long)hq * D, T, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = ti::bf16_map_kpage(&p.map_k, kcache, D, (long long)num_blocks * hkv * 16);
  if (rc) return rc;
  rc = ti::bf16_map_2d(&p.map_v, vcache, 16, (long long)num_blocks * hkv * D, 16, D, CU_TENSOR_MAP_SWIZZLE_32B);
  if (rc) return rc;
  p.block_tables = (const int*)block_tables;
  p.positions = (const int*)positions;
  p.qt_seq = (const int*)qt_seq;
  p.qt_tok0 = (const int*)qt_tok0;
  p.qt_ntok = (const int*)qt_ntok;
  p.gate_src = (const __nv_bfloat16*)gate_src;
  p.out = (__nv_bfloat16*)out;
  p.status = (unsigned*)status;
  p.hq = hq;
  p.hkv = hkv;
  p.max_blocks = max_blocks;
  p.ld = ld;
  p.scale_log2e = scale_log2e;
  cudaStream_t st = (cudaStream_t)stream;
  if (D == 256) return ti::launch_attn_prefill<256>(p, num_tiles, st);
  if (D == 128) return ti::launch_attn_prefill<128>(p, num_tiles, st);
  return ti::launch_attn_prefill<64>(p, num_tiles, st);
}

}  // extern "C"
