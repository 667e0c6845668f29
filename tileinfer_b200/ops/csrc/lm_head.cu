// Sampling front-end on the vocabulary shard of one rank: per-row top-k of the lm_head logits and the
// exchange of the k candidates between tensor-parallel ranks, so that every rank ends up with the
// same tp*k (value, token id) pairs and can sample without a broadcast.
//
// The logits themselves come from the bf16 GEMV (final RMSNorm fused in its prologue, fp32 output).
// Replaces kernels/lm_head_topk.py:6-582 (fused argmax only, indices round-tripped through fp32) and
// the torch.topk + 2x all_gather + rank-0 broadcast of engine/model_runner.py:1012-1083, 879-883.
// Indices stay integers; ties resolve to the smallest token id.
//
// Stage 1: grid (rows, chunks): each block keeps its chunk of the row in registers and extracts the
// k best by repeated block-wide arg-max.  Stage 2: one block per row merges chunks*k candidates the
// same way, then (tp > 1) stores its k winners as tagged packets into every peer's buffer and waits,
// bounded, for the peers' packets.
#include <mutex>

#include "common.cuh"
#include "topk_static.h"

namespace ti {

struct TopkParams {
  const float* logits;           // [M, ld]
  float* ws_val;                 // [M, chunks, k]
  int* ws_idx;                   // [M, chunks, k]
  float* out_val;                // [M, tp*k]
  int* out_idx;                  // [M, tp*k] global token ids
  const unsigned* step_ptr;
  unsigned* status;
  uint64_t peer_buf[kMaxRanks];  // packet buffers [2][tp][m_cap][64] x 16 bytes
  unsigned long long timeout_ns;
  int M, V, ld, k, chunks, chunk_size, vocab_start;
  int tp, rank, order, m_cap;
};

constexpr int kNoIdx = 0x7fffffff;

// Order-preserving key of a float (larger value -> larger key); 0 is reserved for "no element".
TI_DEVICE uint32_t float_key(float v) {
  const uint32_t u = __float_as_uint(v);
  const uint32_t k = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return k == 0u ? 1u : k;
}

// Block-wide top-k (k <= 64) of the EPT elements each of the 256 threads holds, by radix selection: four passes of
// 8 bits narrow down the key of the k-th largest element (a 256-bin histogram in shared memory per pass), then the
// elements above it are compacted, ties at the threshold are taken in position order (the smallest token ids), and
// the k winners are ranked (value descending, token id ascending) and written out.  A dozen block barriers in all,
// where extracting the maxima one by one cost two barriers per extracted element.
// Element e of thread t sits at position t + 256 e; positions are in ascending token-id order among equal values.
struct TopkSmem {
  int hist[256];
  int sel_bin, need, cnt, base;
  int warp_cnt[8];
  float cv[64];
  int ci[64];
};

template <int EPT>
TI_DEVICE void select_topk(float (&val)[EPT], int (&idx)[EPT], int k, float* out_v, int* out_i, TopkSmem& sm) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t key[EPT];
#pragma unroll
  for (int e = 0; e < EPT; ++e) key[e] = idx[e] == kNoIdx ? 0u : float_key(val[e]);
  uint32_t prefix = 0u, mask = 0u;
  int need = k;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    sm.hist[tid] = 0;
    __syncthreads();
#pragma unroll
    for (int e = 0; e < EPT; ++e)
      if ((key[e] & mask) == prefix) atomicAdd(&sm.hist[(key[e] >> shift) & 255u], 1);
    __syncthreads();
    if (warp == 0) {
      // lane l owns bins 255 - 8l .. 248 - 8l; find the bin in which the count from the top reaches `need`
      int c[8], tot = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        c[j] = sm.hist[255 - 8 * lane - j];
        tot += c[j];
      }
      int incl = tot;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const int excl = incl - tot;                         // elements in the bins above this lane's
      if (excl < need && incl >= need) {
        int run = excl;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (run < need && run + c[j] >= need) {
            sm.sel_bin = 255 - 8 * lane - j;
            sm.need = need - run;
          }
          run += c[j];
        }
      }
    }
    __syncthreads();
    prefix |= (uint32_t)sm.sel_bin << shift;
    mask |= 0xFFu << shift;
    need = sm.need;
    __syncthreads();
  }
  // prefix = key of the k-th largest element; `need` of the elements equal to it are taken, everything above it is
  const int n_gt = k - need;
  if (tid == 0) { sm.cnt = 0; sm.base = 0; }
  __syncthreads();
#pragma unroll
  for (int e = 0; e < EPT; ++e)
    if (key[e] > prefix) {
      const int pos = atomicAdd(&sm.cnt, 1);
      sm.cv[pos] = val[e];
      sm.ci[pos] = idx[e];
    }
  // ties in position order: element e of thread t is at position t + 256 e
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const bool tie = key[e] == prefix;
    const unsigned bal = __ballot_sync(0xffffffffu, tie);
    if (lane == 0) sm.warp_cnt[warp] = __popc(bal);
    __syncthreads();
    int before = sm.base, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      if (w < warp) before += sm.warp_cnt[w];
      total += sm.warp_cnt[w];
    }
    const int rank = before + __popc(bal & ((1u << lane) - 1u));
    if (tie && rank < need) {
      sm.cv[n_gt + rank] = key[e] == 0u ? -INFINITY : val[e];
      sm.ci[n_gt + rank] = key[e] == 0u ? -1 : idx[e];
    }
    __syncthreads();
    if (tid == 0) sm.base += total;
    __syncthreads();
    if (sm.base >= need) break;                            // uniform: every thread reads the same value
  }
  __syncthreads();
  // rank the k winners: value descending, then token id ascending (empty entries, id -1, last)
  if (tid < k) {
    const float v = sm.cv[tid];
    const unsigned id = (unsigned)sm.ci[tid];
    int rank = 0;
    for (int j = 0; j < k; ++j) {
      const float vj = sm.cv[j];
      const unsigned ij = (unsigned)sm.ci[j];
      rank += (vj > v || (vj == v && (ij < id || (ij == id && j < tid)))) ? 1 : 0;
    }
    out_v[rank] = v;
    out_i[rank] = (int)id;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(256) topk_stage1_kernel(const __grid_constant__ TopkParams p) {
  constexpr int EPT = 16;
  __shared__ TopkSmem sm;
  const int m = blockIdx.x, c = blockIdx.y;
  pdl_trigger();
  pdl_wait();
  const int lo = c * p.chunk_size, hi = min(p.V, lo + p.chunk_size);
  float val[EPT];
  int idx[EPT];
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const int i = lo + threadIdx.x + e * 256;
    const bool ok = i < hi;
    val[e] = ok ? p.logits[(size_t)m * p.ld + i] : -INFINITY;
    idx[e] = ok ? i : kNoIdx;
  }
  const size_t o = ((size_t)m * p.chunks + c) * p.k;
  select_topk<EPT>(val, idx, p.k, p.ws_val + o, p.ws_idx + o, sm);
}

__global__ void __launch_bounds__(256) topk_stage2_kernel(const __grid_constant__ TopkParams p) {
  constexpr int EPT = 32;
  __shared__ TopkSmem sm;
  __shared__ float fin_v[64];
  __shared__ int fin_i[64];
  const int m = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const int nc = p.chunks * p.k;
  float val[EPT];
  int idx[EPT];
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const int i = threadIdx.x + e * 256;
    const bool ok = i < nc && p.ws_idx[(size_t)m * nc + i] >= 0;
    val[e] = ok ? p.ws_val[(size_t)m * nc + i] : -INFINITY;
    idx[e] = ok ? p.ws_idx[(size_t)m * nc + i] : kNoIdx;
  }
  select_topk<EPT>(val, idx, p.k, fin_v, fin_i, sm);
  __syncthreads();
  const int kk = p.k;
  if (p.tp == 1) {
    for (int j = threadIdx.x; j < kk; j += 256) {
      p.out_val[(size_t)m * kk + j] = fin_v[j];
      p.out_idx[(size_t)m * kk + j] = fin_i[j] < 0 ? -1 : fin_i[j] + p.vocab_start;
    }
    return;
  }
  // ---- candidate all-gather over peer memory: one 16-byte packet pair per candidate
  const unsigned tag = (*p.step_ptr) * 65536u + (unsigned)p.order + 1u;
  const int slot = p.order & 1;
  for (int j = threadIdx.x; j < kk; j += 256) {
    const float v = fin_v[j];
    const int gi = fin_i[j] < 0 ? -1 : fin_i[j] + p.vocab_start;
    const size_t mine = ((((size_t)slot * p.tp + p.rank) * p.m_cap + m) * 64 + j) * 16;
    const size_t cand_bytes = (size_t)2 * p.tp * p.m_cap * 64 * 16;
    jitter();
    if (TI_CHECK(mine + 15, cand_bytes, p.status))
      for (int q = 0; q < p.tp; ++q)
        if (q != p.rank) ll_store2(reinterpret_cast<uint8_t*>(p.peer_buf[q]) + mine, v, __int_as_float(gi), tag);
    const uint8_t* local = reinterpret_cast<const uint8_t*>(p.peer_buf[p.rank]);
    for (int r = 0; r < p.tp; ++r) {
      float a = v, b = __int_as_float(gi);
      if (r != p.rank) {
        const size_t off = ((((size_t)slot * p.tp + r) * p.m_cap + m) * 64 + j) * 16;
        if (TI_CHECK(off + 15, cand_bytes, p.status)) ll_wait2(local + off, tag, a, b, p.timeout_ns, p.status);
      }
      p.out_val[((size_t)m * p.tp + r) * kk + j] = a;
      p.out_idx[((size_t)m * p.tp + r) * kk + j] = __float_as_int(b);
    }
  }
}

}  // namespace ti

extern "C" {

int ti_topk_params_size() { return (int)sizeof(ti::TopkParams); }

int ti_topk(const ti::TopkParams* p, void* stream) {
  if (p->M <= 0) return 0;
  if (p->k < 1 || p->k > 64 || p->chunk_size > 4096 || p->chunks * p->k > 8192) return -2;
  if ((long long)p->chunks * p->chunk_size < p->V) return -3;
  if (p->tp > ti::kMaxRanks || (p->tp > 1 && p->M > p->m_cap)) return -5;
  cudaStream_t st = (cudaStream_t)stream;
  ti::launch_kernel(ti::topk_stage1_kernel, dim3(p->M, p->chunks), dim3(256), 0, st, true, *p);
  ti::launch_kernel(ti::topk_stage2_kernel, dim3(p->M), dim3(256), 0, st, true, *p);
  return (int)cudaGetLastError();
}

// Merge + exchange only: ws_val / ws_idx [M][chunks][k] already hold per-chunk candidates (LOCAL column numbers).
int ti_topk_merge(const ti::TopkParams* p, void* stream) {
  if (p->M <= 0) return 0;
  if (p->k < 1 || p->k > 64 || p->chunks < 1 || p->chunks * p->k > 8192) return -2;
  if (p->tp > ti::kMaxRanks || (p->tp > 1 && p->M > p->m_cap)) return -5;
  cudaError_t e = ti::launch_kernel(ti::topk_stage2_kernel, dim3(p->M), dim3(256), 0, (cudaStream_t)stream, true, *p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // extern "C"

// ------------------------------------------------------------------ allocation-free entry point
// Same two kernels as ti_topk(); the per-chunk candidate workspace is a file-scope device array, so the
// call allocates nothing.  See topk_static.h for who this is for, the limits and the sharing rules.
namespace ti {
static __device__ __align__(256) float g_topk_static_val[TI_TOPK_STATIC_MAX_ENTRIES];
static __device__ __align__(256) int g_topk_static_idx[TI_TOPK_STATIC_MAX_ENTRIES];
constexpr int kMaxDevices = 64;
static float* g_static_val_ptr[kMaxDevices];
static int* g_static_idx_ptr[kMaxDevices];
static std::once_flag g_static_once[kMaxDevices];      // the first calls of two threads on one device do not race
static cudaError_t g_static_err[kMaxDevices];
}  // namespace ti

extern "C" {

const char* ti_topk_static_error(int code) {
  switch (code) {
    case 0: return "ok";
    case -1: return "rows must be in [1, 16]: the static scratch holds 16 rows";
    case -2: return "k must be in [1, 64]";
    case -3: return "vocab must be in [1, 524288] and ld >= vocab";
    case -4: return "null pointer argument";
    case -5: return "more than 64 CUDA devices are not supported";
    case -6: return "logits, out_val and out_idx must be device memory of the CURRENT device (the scratch is per device)";
    default: return code > 0 ? "CUDA error (value is a cudaError_t)" : "unknown error";
  }
}

int ti_topk_static(const float* logits, int rows, int vocab, int ld, int k, int vocab_start, float* out_val,
                   int* out_idx, void* stream) {
  if (logits == nullptr || out_val == nullptr || out_idx == nullptr) return -4;
  if (rows < 1 || rows > TI_TOPK_STATIC_MAX_ROWS) return -1;
  if (k < 1 || k > 64) return -2;
  if (vocab < 1 || vocab > 128 * 4096 || ld < vocab) return -3;
  // chunk geometry: at most 128 chunks and 8192 candidates per row, chunks of a multiple of 256 columns
  const int max_chunks = 8192 / k < 128 ? 8192 / k : 128;
  int cs = (vocab + max_chunks - 1) / max_chunks;
  cs = ((cs + 255) / 256) * 256;
  if (cs < 256) cs = 256;
  if (cs > 4096) return -3;
  const int chunks = (vocab + cs - 1) / cs;
  // the device address of the scratch: the array's name is only a host-side handle, so it is resolved
  // once per device, with that device current, and cached
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= ti::kMaxDevices) return -5;
  // the scratch belongs to the current device: inputs and outputs must live there too (a kernel on this device
  // would otherwise combine another GPU's buffers with this GPU's scratch)
  const void* ptrs[3] = {logits, out_val, out_idx};
  for (const void* q : ptrs) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, q) != cudaSuccess) {
      (void)cudaGetLastError();
      return -6;
    }
    if (at.type == cudaMemoryTypeDevice && at.device != dev) return -6;
  }
  std::call_once(ti::g_static_once[dev], [dev] {
    cudaError_t r = cudaGetSymbolAddress((void**)&ti::g_static_val_ptr[dev], ti::g_topk_static_val);
    if (r == cudaSuccess) r = cudaGetSymbolAddress((void**)&ti::g_static_idx_ptr[dev], ti::g_topk_static_idx);
    ti::g_static_err[dev] = r;
  });
  if (ti::g_static_err[dev] != cudaSuccess) return (int)ti::g_static_err[dev];
  ti::TopkParams p = {};
  p.logits = logits;
  p.ws_val = ti::g_static_val_ptr[dev];
  p.ws_idx = ti::g_static_idx_ptr[dev];
  p.out_val = out_val;
  p.out_idx = out_idx;
  p.M = rows;
  p.V = vocab;
  p.ld = ld;
  p.k = k;
  p.chunks = chunks;
  p.chunk_size = cs;
  p.vocab_start = vocab_start;
  p.tp = 1;
  cudaStream_t st = (cudaStream_t)stream;
  e = ti::launch_kernel(ti::topk_stage1_kernel, dim3(rows, chunks), dim3(256), 0, st, false, p);
  if (e != cudaSuccess) return (int)e;
  e = ti::launch_kernel(ti::topk_stage2_kernel, dim3(rows), dim3(256), 0, st, false, p);
  return (int)e;                         // the launch results only: no stale error of an unrelated earlier call
}

}  // extern "C"
