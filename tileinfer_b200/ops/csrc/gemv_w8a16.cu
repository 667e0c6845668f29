// Skinny W8A16 / bf16 matrix product for decode: y[M<=16, N] = x[M, K] * W[N, K]^T.
//
// Replaces the reference's dequantize_gemv_kernel (kernels/splitk_gemv.py:131-201), which serves
// M == 1 only with 64-bit weight loads, and its M > 1 fallback that re-materialises a bf16 copy of
// the weight for cuBLAS on every call (kernels/splitk_gemv.py:243-247).
//
// Design for sm_100a:
//  * weights are stored as 512-byte tiles [N/8][K/64][8 rows][64 k] (int8) so a warp fetches one
//    tile with a single fully coalesced 128-bit load per lane and keeps 8 such loads in flight;
//  * int8 is widened to bf16 exactly in registers and multiplied on the tensor cores with
//    mma.sync.m16n8k16: activations are the 16-row A operand (one weight pass serves up to 16
//    tokens), the 8 weight rows of the tile are the B operand, accumulation is fp32;
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
};

enum { XGLOBAL = 0, XNORM = 1 };
enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_ROWPAR = 2, EPI_F32 = 3 };
enum { W_INT8 = 0, W_BF16 = 1 };

constexpr int kThreads = 512;
constexpr int kUnroll = 8;

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

template <int WT, int XMODE, int EPI>
TI_DEVICE void gemv_body(const GemvParams& p, int cta, int ncta, uint8_t* smem) {
  constexpr int TK = WT == W_INT8 ? 64 : 32;       // k per 512-byte tile
  constexpr int XW = TK / 4 / 8;                    // 16-byte x loads per tile and token row (2 or 1)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int nwarps = blockDim.x >> 5;
  const bool hi = p.M > 8;
  const int xs_stride = p.K + 8;                    // bf16 elements; +16 bytes keeps LDS.128 conflict-free
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem);

  if (XMODE == XNORM) {
    // ---- RMSNorm(1+w) of up to 16 rows of the residual stream into shared memory
    const int rows = hi ? 16 : 8;
    float* red = reinterpret_cast<float*>(smem + (size_t)rows * xs_stride * 2);   // [nwarps][16]
    const int chunks = p.K >> 3;
    for (int m = 0; m < p.M; ++m) {
      float ss = 0.f;
      for (int c = tid; c < chunks; c += blockDim.x) {
        const uint4 v = ldg_cached16(p.x + (size_t)m * p.ldx + c * 8);
        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = bf16lo(w4[i]), b = bf16hi(w4[i]);
          ss += a * a + b * b;
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) red[warp * 16 + m] = ss;
    }
    __syncthreads();
    for (int m = 0; m < rows; ++m) {
      float rr = 0.f;
      if (m < p.M) {
        float tot = 0.f;
        for (int w = 0; w < nwarps; ++w) tot += red[w * 16 + m];
        rr = rsqrtf(tot / (float)p.K + p.eps);
      }
      for (int c = tid; c < chunks; c += blockDim.x) {
        uint4 o = make_uint4(0, 0, 0, 0);
        if (m < p.M) {
          const uint4 v = ldg_cached16(p.x + (size_t)m * p.ldx + c * 8);
          const uint4 nw = ldg_cached16(p.norm_w + c * 8);
          const uint32_t a4[4] = {v.x, v.y, v.z, v.w}, n4[4] = {nw.x, nw.y, nw.z, nw.w};
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

  const int total_units = p.n_tiles * p.S;
  const int W = ncta * nwarps;
  for (int unit = cta * nwarps + warp; unit < total_units; unit += W) {
    const int nt = unit / p.S, ks = unit - nt * p.S;
    const int kb0 = ks * p.kb_per_split;
    const int kb1 = min(p.KB, kb0 + p.kb_per_split);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const uint8_t* wp = p.w + ((size_t)nt * p.KB + kb0) * 512 + lane * 16;
    for (int kb = kb0; kb < kb1; kb += kUnroll) {
      uint4 wv[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        wv[u] = (kb + u < kb1) ? ldg_stream16(wp + (size_t)u * 512) : make_uint4(0, 0, 0, 0);
      wp += (size_t)kUnroll * 512;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int kbu = min(kb + u, kb1 - 1);
        const int k0 = kbu * TK + t * (TK / 4);
        uint4 xa[XW], ya[XW];
#pragma unroll
        for (int i = 0; i < XW; ++i) {
          if (XMODE == XNORM) {
            xa[i] = *reinterpret_cast<const uint4*>(xs + (size_t)g * xs_stride + k0 + i * 8);
            ya[i] = hi ? *reinterpret_cast<const uint4*>(xs + (size_t)(g + 8) * xs_stride + k0 + i * 8)
                       : make_uint4(0, 0, 0, 0);
          } else {
            xa[i] = (g < p.M) ? ldg_cached16(p.x + (size_t)g * p.ldx + k0 + i * 8) : make_uint4(0, 0, 0, 0);
            ya[i] = (g + 8 < p.M) ? ldg_cached16(p.x + (size_t)(g + 8) * p.ldx + k0 + i * 8) : make_uint4(0, 0, 0, 0);
          }
        }
        const uint32_t ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
        if (WT == W_INT8) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t b0, b1;
            cvt_s8x4_bf16x2(ww[j] ^ 0x80808080u, b0, b1);
            const uint4 xv = xa[j >> 1], yv = ya[j >> 1];
            const uint32_t a0 = (j & 1) ? xv.z : xv.x, a2 = (j & 1) ? xv.w : xv.y;
            const uint32_t a1 = (j & 1) ? yv.z : yv.x, a3 = (j & 1) ? yv.w : yv.y;
            mma_bf16_16816(acc, a0, a1, a2, a3, b0, b1);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const uint32_t b0 = ww[2 * j], b1 = ww[2 * j + 1];
            const uint4 xv = xa[0], yv = ya[0];
            const uint32_t a0 = j ? xv.z : xv.x, a2 = j ? xv.w : xv.y;
            const uint32_t a1 = j ? yv.z : yv.x, a3 = j ? yv.w : yv.y;
            mma_bf16_16816(acc, a0, a1, a2, a3, b0, b1);
          }
        }
      }
    }
    if (p.S == 1) {
      epilogue<EPI>(p, nt, g, t, acc);
    } else {
      *reinterpret_cast<float4*>(p.ws + (size_t)unit * 128 + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      __threadfence();
      __syncwarp();
      unsigned prev = 0;
      if (lane == 0) prev = atomicAdd(p.counters + nt, 1u);
      prev = __shfl_sync(0xffffffffu, prev, 0);
      if (prev == (unsigned)p.S - 1u) {
        __threadfence();
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < p.S; ++s) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(p.ws + ((size_t)nt * p.S + s) * 128 + lane * 4));
          sum[0] += v.x; sum[1] += v.y; sum[2] += v.z; sum[3] += v.w;
        }
        if (lane == 0) p.counters[nt] = 0u;
        epilogue<EPI>(p, nt, g, t, sum);
      }
    }
  }
}

template <int WT, int XMODE, int EPI>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  gemv_body<WT, XMODE, EPI>(p, blockIdx.x, gridDim.x, smem);
}

// All emulated ranks of a tensor-parallel group in ONE cooperative launch on one GPU: block b
// works for rank b / ctas_per_rank.  Used by tests where fewer GPUs than ranks are available;
// separate launches that wait on one another must never share a GPU.
template <int WT, int XMODE, int EPI>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel_ranks(const GemvParams* plist, int ctas_per_rank) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int r = blockIdx.x / ctas_per_rank;
  gemv_body<WT, XMODE, EPI>(plist[r], blockIdx.x - r * ctas_per_rank, ctas_per_rank, smem);
}

static size_t smem_bytes(const GemvParams& p, int xmode) {
  if (xmode != XNORM) return 0;
  const int rows = p.M > 8 ? 16 : 8;
  return (size_t)rows * (p.K + 8) * 2 + (kThreads / 32) * 16 * sizeof(float);
}

template <int WT, int XMODE, int EPI>
static int launch(const GemvParams& p, int ncta, cudaStream_t st, const GemvParams* dev_list, int nranks) {
  const size_t sm = smem_bytes(p, XMODE);
  if (dev_list == nullptr) {
    auto k = gemv_kernel<WT, XMODE, EPI>;
    if (sm > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    k<<<ncta, kThreads, sm, st>>>(p);
  } else {
    auto k = gemv_kernel_ranks<WT, XMODE, EPI>;
    if (sm > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
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

static int check(const GemvParams& p, int wt, int xmode) {
  const int tk = wt == W_INT8 ? 64 : 32;
  if (p.M < 1 || p.M > 16 || p.N < 2 || (p.N & 1) || p.K % tk || p.KB * tk != p.K) return -2;
  if (p.S < 1 || p.kb_per_split < 1 || (long long)p.S * p.kb_per_split < p.KB) return -3;
  if (xmode == XNORM && (p.K % 8 || smem_bytes(p, xmode) > 220 * 1024)) return -4;
  if (p.tp > kMaxRanks || (p.tp > 1 && p.M > p.m_cap)) return -5;
  return 0;
}

}  // namespace ti

extern "C" {

// Launches y = x W^T with the selected weight type, x source and epilogue on `stream`.
// Returns 0 or a CUDA / argument error code.
int ti_gemv(const ti::GemvParams* p, int wt, int xmode, int epi, int ncta, void* stream) {
  int rc = ti::check(*p, wt, xmode);
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
  int rc = ti::check(*p0, wt, xmode);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (wt != ti::W_INT8) return -6;
  return xmode == ti::XNORM ? ti::dispatch_epi<ti::W_INT8, ti::XNORM>(*p0, epi, ncta, st, dev_params, nranks)
                            : ti::dispatch_epi<ti::W_INT8, ti::XGLOBAL>(*p0, epi, ncta, st, dev_params, nranks);
}

int ti_gemv_params_size() { return (int)sizeof(ti::GemvParams); }

}  // extern "C"
